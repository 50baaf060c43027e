"""Where a decode step's time goes: kernel durations and the idle gaps between kernels inside the replayed graph.

    python -m benchmarks.profile_decode --layers 8 --rows 256 --context 700

Builds a Llama-3-70B-shaped model with the per-GPU shapes of 8-way tensor parallelism (``--tp-shape-of``), fills an
eSurge engine with ``--rows`` sequences of ``--context`` tokens, lets the decode graph warm up and be captured, and
then records a few replayed steps with ``torch.profiler`` (CUPTI activity records: these carry start and end time
stamps of every kernel inside the graph). Printed per kernel name: launches per step, mean duration, mean gap since
the previous kernel ended. Durations under the profiler are for attribution, not for quoting; the step time printed
last is taken with CUDA events on un-profiled steps.
"""

from __future__ import annotations

import argparse
import collections

import torch

from easydel_b200.inference import SamplingParams
from easydel_b200.inference.esurge import eSurge
from easydel_b200.inference.esurge.bench_serving import MODELS
from easydel_b200.modules.llama import LlamaConfig, LlamaForCausalLM


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama-3-70b")
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--tp-shape-of", type=int, default=8)
    ap.add_argument("--rows", type=int, default=256)
    ap.add_argument("--context", type=int, default=700)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--timeline", type=int, default=0, help="also list this many consecutive launches in order")
    a = ap.parse_args()
    kw = dict(MODELS[a.model])
    d = a.tp_shape_of
    kw.update(num_hidden_layers=a.layers, num_attention_heads=kw["num_attention_heads"] // d,
              num_key_value_heads=max(1, kw["num_key_value_heads"] // d), intermediate_size=kw["intermediate_size"] // d,
              head_dim=kw["hidden_size"] // kw["num_attention_heads"])
    dev = torch.device("cuda", 0)
    model = LlamaForCausalLM.sequential_init(LlamaConfig(**kw), dtype=torch.bfloat16, param_dtype=torch.bfloat16,
                                             device=dev, seed=1).eval()
    eng = eSurge(model, max_model_len=4096, max_num_seqs=a.rows, max_num_batched_tokens=8192, hbm_utilization=0.5,
                 enable_prefix_caching=False)
    g = torch.Generator().manual_seed(0)
    sp = SamplingParams(max_tokens=64, temperature=0.0, ignore_eos=True)
    for _ in range(a.rows):
        eng.add_request(torch.randint(0, kw["vocab_size"], (a.context,), generator=g).tolist(), sp)
    # prefill everything, then a few decode steps so that the bucket's graph exists
    while eng.scheduler.num_waiting or eng.runner.timings["graph_steps"] < 4:
        eng.step()
    torch.cuda.synchronize()
    eng.runner.time_decode_steps = True
    for _ in range(8):
        eng.step()
    times = eng.runner.decode_step_times()
    eng.runner.time_decode_steps = False
    from torch.profiler import ProfilerActivity, profile

    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(a.steps):
            eng.step()
        torch.cuda.synchronize()
    evs = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA and e.time_range.end >
                  e.time_range.start),
                 key=lambda e: e.time_range.start)
    dur, gap, cnt = collections.Counter(), collections.Counter(), collections.Counter()
    prev_end = None
    for e in evs:
        name = e.name.replace("(anonymous namespace)::", "").replace("void ", "").split("(")[0][:70]
        dur[name] += e.time_range.end - e.time_range.start
        if prev_end is not None:
            gap[name] += max(0.0, min(e.time_range.start - prev_end, 50.0))    # cap: step boundaries are not gaps
        cnt[name] += 1
        prev_end = max(prev_end or 0, e.time_range.end)
    if a.timeline:
        # one layer's worth of launches in order, from the middle of the last recorded step
        mid = len(evs) - len(evs) // (2 * a.steps)
        t_ref = evs[mid].time_range.start
        print("timeline (us since the first listed kernel started): start, duration, name")
        for e in evs[mid:mid + a.timeline]:
            print(f"  {e.time_range.start - t_ref:9.2f} {e.time_range.end - e.time_range.start:8.2f}  "
                  f"{e.name.replace('(anonymous namespace)::', '').replace('void ', '').split('(')[0][:90]}")
    total_d, total_g = sum(dur.values()), sum(gap.values())
    print(f"{'kernel':70s} {'per step':>8s} {'dur us':>8s} {'gap us':>8s} {'share':>6s}")
    for name, _ in sorted(dur.items(), key=lambda kv: -kv[1] - gap[kv[0]]):
        n = cnt[name]
        print(f"{name:70s} {n / a.steps:8.1f} {dur[name] / n:8.2f} {gap[name] / n:8.2f} "
              f"{(dur[name] + gap[name]) / (total_d + total_g):6.1%}")
    print(f"per step under the profiler: kernels {total_d / a.steps / 1e3:.3f} ms + gaps {total_g / a.steps / 1e3:.3f} ms")
    for bp, v in sorted(times.items()):
        v = sorted(v)
        print(f"decode step without the profiler, {bp} rows, {a.layers} layers: median {v[len(v) // 2]:.3f} ms "
              f"({v[len(v) // 2] / a.layers * 1e3:.1f} us per layer incl. head and sampler)")
    eng.close()


if __name__ == "__main__":
    main()
