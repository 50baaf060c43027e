"""Checkpoint layout and round trips: save_pretrained / from_pretrained, save_state / resume, HF safetensors import."""

import json
import os

import torch

from easydel_b200.infra.base_state import EasyDeLState
from easydel_b200.io import zarr_store as Z
from easydel_b200.modules.auto import AutoEasyDeLModelForCausalLM
from easydel_b200.modules.llama import LlamaConfig, LlamaForCausalLM
from easydel_b200.optimizers import OptimizerFactory, SchedulerConfig
from easydel_b200.trainers import Trainer, TrainingArguments


def _model(seed=0):
    cfg = LlamaConfig(vocab_size=256, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=64)
    torch.manual_seed(seed)
    return LlamaForCausalLM(cfg, dtype=torch.float32, param_dtype=torch.float32)


def test_zarr_array_roundtrip_dtypes_and_chunks(tmp_path):
    for dt in (torch.float32, torch.bfloat16, torch.int64, torch.float16):
        t = (torch.randn(37, 50) * 10).to(dt)
        Z.write_array(str(tmp_path / f"a_{dt}"), t, chunks=[16, 32])
        back = Z.read_array(str(tmp_path / f"a_{dt}"))
        assert back.dtype == dt and torch.equal(back, t)
    meta = Z.read_meta(str(tmp_path / f"a_{torch.bfloat16}"))
    assert meta["dtype"] == "bfloat16" and meta["zarr_format"] == 2 and meta["compressor"]["id"] == "zstd"
    s = torch.tensor(3.5)
    Z.write_array(str(tmp_path / "s"), s)
    assert Z.read_array(str(tmp_path / "s")).item() == 3.5


def test_save_pretrained_layout_and_reload(tmp_path):
    m = _model()
    d = str(tmp_path / "ckpt")
    m.save_pretrained(d)
    for f in ("config.json", "generation_config.json", "README.md", "tensorstore_index.json",
              "checkpoint_metadata.json"):
        assert os.path.exists(os.path.join(d, f)), f
    idx = json.load(open(os.path.join(d, "tensorstore_index.json")))
    assert idx["format"] == "tensorstore" and idx["version"] == "easydel"
    paths = {e["path"]: e for e in idx["prefixes"]["model"]}
    # reference leaf naming: transposed kernels, embedding leaf, unfused q/k/v
    assert paths["model/model/layers/0/self_attn/q_proj/kernel"]["shape"] == [64, 64]
    assert paths["model/model/layers/0/self_attn/k_proj/kernel"]["shape"] == [64, 32]
    assert paths["model/model/layers/0/mlp/gate_proj/kernel"]["shape"] == [64, 128]
    assert paths["model/model/embed_tokens/embedding"]["shape"] == [256, 64]
    assert paths["model/model/norm/kernel"]["shape"] == [64]
    assert paths["model/lm_head/kernel"]["shape"] == [64, 256]
    assert os.path.exists(os.path.join(d, "model/model/layers/0/self_attn/q_proj/kernel/.zarray"))
    cfg = json.load(open(os.path.join(d, "config.json")))
    assert cfg["model_type"] == "llama" and cfg["architectures"] == ["LlamaForCausalLM"]
    assert "attn_dtype" not in cfg
    m2 = AutoEasyDeLModelForCausalLM.from_pretrained(d, dtype=torch.float32, device="cpu")
    ids = torch.randint(0, 256, (2, 16))
    with torch.no_grad():
        assert torch.allclose(m(input_ids=ids).logits, m2(input_ids=ids).logits, atol=1e-6)


def test_state_save_resume_continues_identically(tmp_path):
    ids = torch.randint(0, 256, (4, 32), generator=torch.Generator().manual_seed(1))

    def run(model, state, n):
        losses = []
        for _ in range(n):
            _, met = model.compute_loss(input_ids=ids, labels=ids)
            met.loss.backward()
            state.apply_gradients()
            losses.append(met.loss.item())
        return losses

    def tx():
        return OptimizerFactory.create("adamw", SchedulerConfig("cosine", learning_rate=1e-3, steps=10,
                                                                warmup_steps=2), weight_decay=0.01)[0]

    m_a = _model()
    s_a = EasyDeLState.create(model=m_a, tx=tx(), init_opt_state=True)
    ref = run(m_a, s_a, 6)
    m_b = _model()
    s_b = EasyDeLState.create(model=m_b, tx=tx(), init_opt_state=True)
    first = run(m_b, s_b, 3)
    d = str(tmp_path / "run-3")
    s_b.save_state(d)
    meta = json.load(open(os.path.join(d, "metadata.json")))
    assert meta["step"] == 3 and meta["has_optimizer_state"]
    idx = json.load(open(os.path.join(d, "tensorstore_index.json")))
    assert "tx" in idx["prefixes"] and any(e["path"].startswith("tx/mu/") for e in idx["prefixes"]["tx"])
    s_c = EasyDeLState.load_state(d, model_class=LlamaForCausalLM, tx_template=tx(), dtype=torch.float32,
                                  device="cpu")
    assert s_c.step == 3
    s_c.model.train()
    rest = run(s_c.model, s_c, 3)
    assert max(abs(a - b) for a, b in zip(ref, first + rest)) < 1e-5


def test_trainer_resumes_from_latest_run(tmp_path):
    g = torch.Generator().manual_seed(0)
    base = torch.randint(0, 256, (4, 32), generator=g)
    data = [{"input_ids": base[i % 4], "labels": base[i % 4]} for i in range(16)]
    kw = dict(model_name="m", save_directory=str(tmp_path), total_batch_size=4, learning_rate=1e-3, use_wandb=False,
              progress_bar_type="none", shuffle_train_dataset=False, num_train_epochs=2, report_steps=1)
    t1 = Trainer(arguments=TrainingArguments(max_training_steps=4, save_steps=2, save_total_limit=1, **kw),
                 model=_model(), dataset_train=data)
    out1 = t1.train()
    assert out1.state.step == 4 and os.path.isdir(os.path.join(str(tmp_path), "m", "run-4"))
    assert not os.path.isdir(os.path.join(str(tmp_path), "m", "run-2"))  # save_total_limit
    assert os.path.exists(os.path.join(str(tmp_path), "m", "run-4", "easydel-training-arguments.json"))
    t2 = Trainer(arguments=TrainingArguments(max_training_steps=6, do_last_save=False, **kw), model=_model(seed=5),
                 dataset_train=data)
    assert t2.model_state.step == 4 and t2._resumed_from.endswith("run-4")
    for (n, a), (_, b) in zip(out1.state.model.named_parameters(), t2.model.named_parameters()):
        assert torch.allclose(a, b), n
    out2 = t2.train()
    assert out2.state.step == 6


def test_hf_safetensors_import(tmp_path):
    from safetensors.torch import save_file

    from easydel_b200.utils.parameters_transformation import internal_to_hf

    m = _model()
    d = tmp_path / "hf"
    d.mkdir()
    save_file({k: v.contiguous() for k, v in internal_to_hf(m).items()}, str(d / "model.safetensors"))
    m.config.save_pretrained(str(d))
    m2 = AutoEasyDeLModelForCausalLM.from_pretrained(str(d), dtype=torch.float32, device="cpu")
    ids = torch.randint(0, 256, (1, 8))
    with torch.no_grad():
        assert torch.allclose(m(input_ids=ids).logits, m2(input_ids=ids).logits, atol=1e-6)


def test_streaming_hf_conversion_matches_in_memory_load(tmp_path):
    """A sharded Hugging Face safetensors checkpoint (dense and MoE) converted tensor by tensor: the EasyDeL
    directory loads into the same logits as loading the safetensors directly, and no more than one stacked expert
    projection was ever held."""
    import json
    import os

    from safetensors.torch import save_file

    from easydel_b200.infra.factory import TaskType, registry
    from easydel_b200.io.streaming_convert import LazySafetensors, stream_hf_to_easydel
    from easydel_b200.utils.parameters_transformation import internal_to_hf
    import easydel_b200.modules  # noqa: F401

    for mtype, extra in (("llama", {}), ("qwen3_moe", dict(num_experts=4, num_experts_per_tok=2,
                                                          moe_intermediate_size=32, head_dim=16))):
        cfg = registry.get_config(mtype)(vocab_size=128, hidden_size=64, intermediate_size=96, num_hidden_layers=2,
                                         num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=64,
                                         **extra)
        reg = registry.get_module_registration(TaskType.CAUSAL_LM, mtype)
        torch.manual_seed(0)
        model = reg.module(cfg, dtype=torch.float32, param_dtype=torch.float32).eval()
        assert model.can_generate()
        src = tmp_path / f"{mtype}_hf"
        os.makedirs(src)
        sd = {k: v.detach().contiguous().clone() for k, v in internal_to_hf(model).items()}
        keys = sorted(sd)
        half = len(keys) // 2
        shards = {"model-00001-of-00002.safetensors": keys[:half], "model-00002-of-00002.safetensors": keys[half:]}
        for fn, ks in shards.items():
            save_file({k: sd[k] for k in ks}, str(src / fn), metadata={"format": "pt"})
        with open(src / "model.safetensors.index.json", "w") as f:
            json.dump({"metadata": {}, "weight_map": {k: fn for fn, ks in shards.items() for k in ks}}, f)
        model.config.save_pretrained(str(src))
        lazy = LazySafetensors(str(src))
        assert len(lazy) == len(sd) and lazy.reads == 0
        lazy.close()
        out = tmp_path / f"{mtype}_ed"
        stats = stream_hf_to_easydel(str(src), str(out), dtype=torch.float32)
        biggest = max(v.numel() * 4 for v in model.state_dict().values())
        assert stats["tensors"] > 0 and stats["peak_tensor_bytes"] <= biggest
        assert os.path.exists(out / "tensorstore_index.json") and os.path.exists(out / "config.json")
        back = reg.module.from_pretrained(str(out), dtype=torch.float32, device="cpu")
        ids = torch.randint(0, 128, (1, 12), generator=torch.Generator().manual_seed(1))
        with torch.no_grad():
            assert torch.allclose(back(input_ids=ids).logits, model(input_ids=ids).logits, atol=1e-5)
