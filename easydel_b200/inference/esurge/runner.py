"""Model runner: turns a ``SchedulerOutput`` into one device step and returns the sampled tokens.

Role of ``eSurgeRunner`` / ``ExecutionManager`` / ``BatchMetadataPreparer`` in the reference
(easydel/inference/esurge/runners/*): per step one packed host->device upload of the ragged-batch
metadata, the backbone over the flattened tokens with the paged cache, the LM head on each
sequence's last position only, the sampler, and one small device->host download of the tokens.
Instead of ahead-of-time compiled buckets the step is eager kernel launches on persistent,
fixed-size device buffers (so that decode steps can be replayed from CUDA graphs).
"""

from __future__ import annotations

import time
import typing as tp

import numpy as np
import torch

from ...caching.paged import PAGE_SIZE, PagedBatchMeta, PagedKVCache
from ...ops import functional as F
from ...ops import serving as S
from .scheduler import SchedulerOutput


class ModelRunner:
    def __init__(self, model, cache: PagedKVCache, max_num_seqs: int, max_num_batched_tokens: int,
                 max_model_len: int):
        self.model = model
        # a vision-language wrapper is served through its language model; image rows arrive as embeddings
        self._lm = getattr(model, "language_model", model)
        self.cache = cache
        self.device = model.device
        self.max_num_seqs = max_num_seqs
        self.max_tokens = max_num_batched_tokens
        self.max_pages_per_seq = (max_model_len + PAGE_SIZE - 1) // PAGE_SIZE
        self.vocab = model.spec.vocab_size
        dev = self.device
        pin = dev.type == "cuda"
        B, T, MP = max_num_seqs, max_num_batched_tokens, self.max_pages_per_seq
        # one packed int32 staging buffer: ids | pos | slots | cu_q | kv_lens | last_idx | page_table |
        # slot of every sequence | (token row, slot) of the rows whose input token is still on the device
        self._sizes = [T, T, T, B + 1, B, B, B * MP, B, B, B]
        # cache groups beyond the first (window-bounded layers with their own pools): slot mapping + page table each
        self.num_groups = getattr(cache, "num_groups", 1)
        for _ in range(self.num_groups - 1):
            self._sizes += [T, B * MP]
        # models that rotate with three position streams (vision tokens at grid coordinates): [3, T] rotary positions
        # beside the token indices, which keep addressing the cache
        cfg = getattr(model.config, "text_config", None) or model.config
        rs = getattr(cfg, "rope_scaling", None) or getattr(model.config, "rope_scaling", None) or {}
        self.rope3 = isinstance(rs, dict) and "mrope_section" in rs
        self._rope_idx = len(self._sizes) if self.rope3 else -1
        if self.rope3:
            self._sizes.append(3 * T)
        total = sum(self._sizes)
        self._host = torch.zeros(total, dtype=torch.int32, pin_memory=pin)
        self._dev = torch.zeros(total, dtype=torch.int32, device=dev)
        self._hviews = self._split(self._host)
        self._dviews = self._split(self._dev)
        # per-row sampling parameters (float and int blocks)
        self._fhost = torch.zeros(6 * B, dtype=torch.float32, pin_memory=pin)
        self._fdev = torch.zeros(6 * B, dtype=torch.float32, device=dev)
        self._ihost = torch.zeros(3 * B, dtype=torch.int64, pin_memory=pin)
        self._idev = torch.zeros(3 * B, dtype=torch.int64, device=dev)
        # host mirror of every slot's page list, so that decode steps are filled without per-request slicing
        self._slot_pages = np.zeros((B, MP), dtype=np.int32)
        self._slot_npages = np.zeros(B, dtype=np.int32)
        self._slot_epoch = np.full(B, -1, dtype=np.int64)
        try:
            from ...data import _native

            self._native = _native._lib()
        except Exception:
            self._native = None
        self.counts: torch.Tensor | None = None
        self.timings: dict[str, float] = {"prep": 0.0, "exec": 0.0, "sample": 0.0, "d2h": 0.0, "steps": 0,
                                          "graph_steps": 0}
        # The last token sampled for every engine slot stays on the device: a step launched before the previous
        # step's tokens were read back takes its decode inputs from here (asynchronous scheduling).
        self._last_tokens = torch.zeros(B + 1, dtype=torch.int64, device=dev)
        # two read-back buffers, used alternately: [tokens of up to B rows | kernel status word]
        self._tok_host = [torch.zeros(B + 1, dtype=torch.int64, pin_memory=pin) for _ in range(2)]
        self._tok_dev = torch.zeros(B + 1, dtype=torch.int64, device=dev)
        self._launches = 0
        # Decode-only greedy steps are replayed from CUDA graphs, one per power-of-two batch bucket
        # (the reference compiles (tokens, requests) buckets ahead of time: runners/execution_manager.py:1291-1405).
        import os

        self.use_graphs = dev.type == "cuda" and os.environ.get("EDL_ESURGE_CUDA_GRAPHS", "1") != "0"
        latent_kernel = bool(cache.latent and cache.k.shape[-1] == 576)    # the 512 + 64 layout has a decode kernel
        if cache.linear or getattr(cache, "compressed", False) or (cache.latent and not latent_kernel) or \
                (not cache.latent and model.spec.head_dim not in (64, 128)):
            self.use_graphs = False     # these serving paths are tensor code with host-side steps: run eagerly
        self._seq_slots = torch.zeros(max_num_seqs, dtype=torch.int64, device=dev)
        self._graphs: dict[int, tuple[tp.Any, torch.Tensor]] = {}
        # device time of replayed decode steps (CUDA events around the graph launch), read by decode_step_times()
        self.time_decode_steps = False
        self._step_events: list = []
        self._graph_pool = None
        self._warm: set[int] = set()
        self._sms = torch.cuda.get_device_properties(dev).multi_processor_count if dev.type == "cuda" else 1
        self.tp_group = None
        mesh = getattr(model.config, "mesh", None)
        if mesh is not None and getattr(mesh, "tp", 1) > 1:
            self.tp_group = mesh.get_group("tp")

    def decode_step_times(self) -> dict[int, list[float]]:
        """Milliseconds on the device of every replayed decode step recorded since the last call, by batch bucket
        (``time_decode_steps`` must be on). Synchronises the device."""
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        out: dict[int, list[float]] = {}
        for bp, e0, e1 in self._step_events:
            out.setdefault(bp, []).append(e0.elapsed_time(e1))
        self._step_events = []
        return out

    def release(self) -> None:
        """Drops the captured graphs (and with them their private memory pool). Needed before the process group
        is torn down: a graph that holds collectives keeps the communicator's resources alive."""
        self._graphs.clear()
        self._graph_pool = None
        self._warm.clear()
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)

    def _split(self, buf: torch.Tensor) -> list[torch.Tensor]:
        out, o = [], 0
        for n in self._sizes:
            out.append(buf[o:o + n])
            o += n
        return out

    # ------------------------------------------------------------------
    def _ensure_counts(self) -> torch.Tensor:
        if self.counts is None:
            self.counts = torch.zeros(self.max_num_seqs, self.vocab, dtype=torch.int32, device=self.device)
        return self.counts

    def reset_slot(self, slot: int, token_ids: tp.Sequence[int] | None = None) -> None:
        """Clears (and re-seeds) the penalty counts of a slot when a request takes it."""
        if self.counts is None:
            return
        self.counts[slot].zero_()
        if token_ids:
            t = torch.tensor(list(token_ids), dtype=torch.int64, device=self.device)
            self.counts[slot].index_put_((t,), torch.ones_like(t, dtype=torch.int32), accumulate=True)

    def _decode_splits(self, B: int) -> int:
        """Key-range splits for a decode step of ``B`` rows: enough (row, kv-head, split) units to fill the SMs."""
        if self.device.type != "cuda" or self.max_pages_per_seq < 8:
            return 1
        units = B * max(1, self.cache.num_kv_heads)
        if units * 2 > self._sms:
            return 1
        return int(min(8, self.max_pages_per_seq // 4, max(1, self._sms // units)))

    def _forward(self, B: int, T: int, max_q: int, num_decode: int, mm_rows=None) -> torch.Tensor:
        """Backbone over the first ``T`` staged tokens of ``B`` sequences, LM head on each sequence's last row.
        ``mm_rows``: ``[(first staged row, features [n, hidden])]`` to write over the token embeddings."""
        d_ids, d_pos, d_slots, d_cu, d_kv, d_last, d_table = self._dviews[:7]
        MP = self.max_pages_per_seq
        meta = PagedBatchMeta(cu_q=d_cu[:B + 1], kv_lens=d_kv[:B], page_table=d_table.view(self.max_num_seqs, MP)[:B],
                              slot_mapping=d_slots[:T], max_q=max_q, num_seqs=B, last_token_index=d_last[:B],
                              request_distribution=(num_decode, B, B),
                              num_splits=self._decode_splits(B) if (max_q == 1 and T == B) else 1,
                              seq_slots=self._seq_slots[:B] if self.cache.linear else None)
        if self.num_groups > 1:
            extra = self._dviews[10:]
            meta.group_slots = [extra[2 * g][:T] for g in range(self.num_groups - 1)]
            meta.group_tables = [extra[2 * g + 1].view(self.max_num_seqs, MP)[:B] for g in range(self.num_groups - 1)]
        self.cache.step_meta = meta
        model = self._lm
        if self.rope3:
            d_pos = self._dviews[self._rope_idx].view(3, self.max_tokens)[:, :T][:, None, :]   # [3, 1, T]
        else:
            d_pos = d_pos[:T][None]
        if mm_rows:
            emb = model.get_input_embeddings()(d_ids[:T].long())
            for row0, feats in mm_rows:
                emb[row0:row0 + feats.shape[0]] = feats.to(emb.dtype)
            res = model(inputs_embeds=emb[None], position_ids=d_pos, past_key_values=self.cache,
                        cache_metadata=meta, apply_lm_head=False)
        else:
            res = model(input_ids=d_ids[:T][None].long(), position_ids=d_pos, past_key_values=self.cache,
                        cache_metadata=meta, apply_lm_head=False)
        rows = S.gather_rows(res.last_hidden_state[0], d_last[:B])
        if self.tp_group is not None and hasattr(model, "apply_lm_head_vocab_parallel"):
            return model.apply_lm_head_vocab_parallel(rows, self.tp_group)
        return model.apply_lm_head(rows)

    def _fill_extra_groups(self, sched, B: int) -> None:
        """Slot mapping and page table of the cache groups beyond the first, from every request's per-group page
        list (same indexing by position as group 0; pages a window no longer reaches are the null page)."""
        MP = self.max_pages_per_seq
        for g in range(self.num_groups - 1):
            slots_np = self._hviews[10 + 2 * g].numpy()
            table_np = self._hviews[11 + 2 * g].numpy().reshape(self.max_num_seqs, MP)
            o = 0
            for b, s in enumerate(sched):
                pg = np.asarray(s.request.group_pages[g], dtype=np.int32)
                n, st = s.num_new_tokens, s.start
                if n == 1:
                    slots_np[o] = pg[st >> 7] * PAGE_SIZE + (st & (PAGE_SIZE - 1))
                else:
                    p = np.arange(st, st + n, dtype=np.int32)
                    slots_np[o:o + n] = pg[p // PAGE_SIZE] * PAGE_SIZE + p % PAGE_SIZE
                table_np[b, :len(pg)] = pg
                o += n

    def _decode_step_graphed(self, Bp: int) -> torch.Tensor:
        """Greedy decode step for ``Bp`` rows: eager the first time (warm-up), captured the second, replayed after."""
        entry = self._graphs.get(Bp)
        if entry is not None:
            entry[0].replay()
            return entry[1]
        if Bp not in self._warm:
            self._warm.add(Bp)
            return S.sample(self._forward(Bp, Bp, 1, Bp))[0]
        torch.cuda.synchronize(self.device)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, pool=self._graph_pool):
            toks = S.sample(self._forward(Bp, Bp, 1, Bp))[0]
        if self._graph_pool is None:
            self._graph_pool = g.pool()
        self._graphs[Bp] = (g, toks)
        g.replay()
        return toks

    @torch.no_grad()
    def execute(self, out: SchedulerOutput) -> dict[str, int]:
        """Runs one engine step; returns ``{request_id: sampled token}`` for the requests that sampled."""
        handle = self.launch(out)
        return self.collect(handle) if handle is not None else {}

    def collect(self, handle) -> dict[str, int]:
        """Waits for a launched step and returns its tokens. Also the point where a kernel whose bounded wait ran
        out is noticed: its status word travels with the tokens."""
        t3 = time.perf_counter()
        sched, B, buf, event = handle
        if event is not None:
            event.synchronize()
        host = buf[:B + 1].tolist()
        self.timings["d2h"] += time.perf_counter() - t3
        if host[B] != 0:
            from ...ops import _lib

            _lib.status_word(self.device).zero_()
            raise RuntimeError(f"a kernel of this engine step reported status {host[B]} (a bounded wait ran out); "
                               "the step's output is not valid")
        return {s.request.request_id: host[b] for b, s in enumerate(sched) if s.samples}

    @torch.no_grad()
    def launch(self, out: SchedulerOutput):
        """Enqueues one engine step on the device and returns a handle for :meth:`collect`; does not wait for it."""
        t0 = time.perf_counter()
        sched = out.scheduled
        B = len(sched)
        T = out.total_tokens
        if B == 0:
            return None
        if B > self.max_num_seqs or T > self.max_tokens:
            raise RuntimeError(f"batch of {B} sequences / {T} tokens exceeds the runner's buffers")
        ids, pos, slots, cu_q, kv_lens, last_idx, table, slot_of, fix_pos, fix_slot = self._hviews[:10]
        slotof_np, fixpos_np, fixslot_np = slot_of.numpy(), fix_pos.numpy(), fix_slot.numpy()
        nfix = 0
        MP = self.max_pages_per_seq
        ids_np, pos_np, slots_np = ids.numpy(), pos.numpy(), slots.numpy()
        table_np = table.numpy().reshape(self.max_num_seqs, MP)
        cu_np, kv_np, last_np = cu_q.numpy(), kv_lens.numpy(), last_idx.numpy()
        rope_np = self._hviews[self._rope_idx].numpy().reshape(3, self.max_tokens) if self.rope3 else None
        o = 0
        max_q = 0
        cu_np[0] = 0
        any_pen = False
        any_random = False
        mm_rows = []
        fast = all(s.num_new_tokens == 1 and s.start >= s.request.num_prompt_tokens for s in sched)
        if fast:
            # Decode-only step: vectorised fill from the per-slot page mirror (one short Python pass per field).
            sp_pages, sp_n = self._slot_pages, self._slot_npages
            slot_idx = np.fromiter((s.request.slot for s in sched), dtype=np.int64, count=B)
            for s in sched:   # pages only grow by one every 128 tokens: this loop rarely copies anything
                req = s.request
                n_pg = len(req.pages)
                if sp_n[req.slot] != n_pg or self._slot_epoch[req.slot] != req.pages_epoch:
                    sp_pages[req.slot, :n_pg] = req.pages
                    sp_n[req.slot] = n_pg
                    self._slot_epoch[req.slot] = req.pages_epoch
                sp = req.sampling_params
                any_pen |= sp.needs_penalties
                any_random |= not sp.is_greedy
            p = np.fromiter((s.start for s in sched), dtype=np.int32, count=B)
            ids_np[:B] = np.fromiter((s.request.output_token_ids[-1] for s in sched), dtype=np.int32, count=B)
            pos_np[:B] = p
            if rope_np is not None:
                rope_np[:, :B] = p + np.fromiter((s.request.rope_delta for s in sched), dtype=np.int32, count=B)
            slotof_np[:B] = slot_idx
            on_dev = np.nonzero(ids_np[:B] < 0)[0]          # tokens sampled by a step that was not read back yet
            nfix = len(on_dev)
            if nfix:
                fixpos_np[:nfix] = on_dev
                fixslot_np[:nfix] = slot_idx[on_dev]
                ids_np[on_dev] = 0
            if self._native is not None:     # one C++ pass over the rows (csrc/host_native.cu)
                self._native.edl_host_fill_decode(slot_idx.ctypes.data, p.ctypes.data, B, sp_pages.ctypes.data, MP,
                                                  PAGE_SIZE, slots_np.ctypes.data, table_np.ctypes.data,
                                                  kv_np.ctypes.data, cu_np.ctypes.data, last_np.ctypes.data)
            else:
                rows = sp_pages[slot_idx]
                slots_np[:B] = rows[np.arange(B), p >> 7] * PAGE_SIZE + (p & (PAGE_SIZE - 1))
                table_np[:B] = rows
                kv_np[:B] = p + 1
                cu_np[:B + 1] = np.arange(B + 1, dtype=np.int32)
                last_np[:B] = np.arange(B, dtype=np.int32)
            max_q = 1
        for b, s in enumerate(sched if not fast else ()):
            req = s.request
            n, st = s.num_new_tokens, s.start
            npt = req.num_prompt_tokens
            if st + n <= npt:
                toks = req.prompt_token_ids[st:st + n]
            elif st >= npt:
                toks = req.output_token_ids[st - npt:st - npt + n]
            else:
                toks = req.prompt_token_ids[st:] + req.output_token_ids[:st + n - npt]
            ids_np[o:o + n] = toks
            slotof_np[b] = req.slot if req.slot >= 0 else self.max_num_seqs
            if toks[-1] < 0:       # the one token a decoding row feeds may still be on the device
                fixpos_np[nfix], fixslot_np[nfix] = o + n - 1, req.slot
                ids_np[o + n - 1] = 0
                nfix += 1
            for off, feats in req.mm_embeds:
                # the part of this image that falls inside [st, st + n): chunked prefill may split an image
                a, z = max(off, st), min(off + feats.shape[0], st + n)
                if a < z:
                    mm_rows.append((o + a - st, feats[a - off:z - off]))
            p = np.arange(st, st + n, dtype=np.int32)
            pos_np[o:o + n] = p
            if rope_np is not None:
                rope_np[:, o:o + n] = p + req.rope_delta
                if req.rope_positions is not None and st < npt:       # prompt tokens carry their grid positions
                    z = min(st + n, npt)
                    rope_np[:, o:o + z - st] = req.rope_positions[:, st:z]
            pg = np.asarray(req.pages, dtype=np.int32)
            slots_np[o:o + n] = pg[p // PAGE_SIZE] * PAGE_SIZE + p % PAGE_SIZE
            table_np[b, :len(pg)] = pg
            if req.slot >= 0:
                self._slot_pages[req.slot, :len(pg)] = pg
                self._slot_npages[req.slot] = len(pg)
                self._slot_epoch[req.slot] = req.pages_epoch
            kv_np[b] = st + n
            o += n
            cu_np[b + 1] = o
            last_np[b] = o - 1
            max_q = max(max_q, n)
            sp = req.sampling_params
            any_pen |= sp.needs_penalties
            any_random |= not sp.is_greedy
        if self.num_groups > 1:
            self._fill_extra_groups(sched, B)
        decode_only = max_q == 1 and not any_pen and not any_random
        Bp = B
        if self.use_graphs and decode_only:
            Bp = 1
            while Bp < B:
                Bp *= 2
            Bp = min(Bp, self.max_num_seqs)
            if Bp > B:   # pad rows: token 0 at position 0 written to the null page, attending to one key
                ids_np[B:Bp] = 0
                pos_np[B:Bp] = 0
                if rope_np is not None:
                    rope_np[:, B:Bp] = 0
                slots_np[B:Bp] = 0
                table_np[B:Bp, :] = 0
                kv_np[B:Bp] = 1
                cu_np[B + 1:Bp + 1] = np.arange(B + 1, Bp + 1, dtype=np.int32)
                last_np[B:Bp] = np.arange(B, Bp, dtype=np.int32)
                slotof_np[B:Bp] = self.max_num_seqs
                for g in range(self.num_groups - 1):
                    self._hviews[10 + 2 * g].numpy()[B:Bp] = 0
                    self._hviews[11 + 2 * g].numpy().reshape(self.max_num_seqs, MP)[B:Bp, :] = 0
        if self.cache.linear:
            # recurrent-state rows of the scheduled sequences; padding rows of a batch bucket share the spare row
            sl = [s.request.slot for s in sched] + [self.max_num_seqs] * (Bp - B)
            self._seq_slots[:Bp].copy_(torch.tensor(sl, dtype=torch.int64), non_blocking=True)
        # one upload of the packed metadata
        self._dev.copy_(self._host, non_blocking=True)
        if nfix:
            d_fixpos, d_fixslot = self._dviews[8][:nfix].long(), self._dviews[9][:nfix].long()
            self._dviews[0].index_copy_(0, d_fixpos, self._last_tokens.index_select(0, d_fixslot).to(torch.int32))
        t1 = time.perf_counter()
        from ...utils.helpers import nvtx_range

        with nvtx_range(f"esurge_step_B{B}_T{T}"):
            tokens, t2, t3 = self._run_model(out, sched, B, Bp, T, max_q, decode_only, any_pen, any_random, mm_rows)
        return self._finish_launch(sched, B, tokens, t0, t1, t2, t3)

    def _run_model(self, out, sched, B, Bp, T, max_q, decode_only, any_pen, any_random, mm_rows):
        if self.use_graphs and decode_only:
            if self.time_decode_steps and Bp in self._graphs:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                tokens = self._decode_step_graphed(Bp)[:B]
                e1.record()
                self._step_events.append((Bp, e0, e1))
            else:
                tokens = self._decode_step_graphed(Bp)[:B]
            self.timings["graph_steps"] += 1
            t2 = time.perf_counter()
        else:
            logits = self._forward(B, T, max_q, out.num_decode, mm_rows)
            t2 = time.perf_counter()
            kw = {}
            if any_random or any_pen:
                fh, ih = self._fhost.view(6, -1), self._ihost.view(3, -1)
                for b, s in enumerate(sched):
                    sp = s.request.sampling_params
                    fh[0, b] = 0.0 if sp.is_greedy else sp.temperature
                    fh[1, b], fh[2, b] = sp.top_p, sp.min_p
                    fh[3, b], fh[4, b], fh[5, b] = sp.presence_penalty, sp.frequency_penalty, sp.repetition_penalty
                    ih[0, b] = sp.top_k
                    ih[1, b] = sp.seed if sp.seed is not None else hash(s.request.request_id) & 0x7FFFFFFF
                    ih[2, b] = len(s.request.output_token_ids)
                self._fdev.copy_(self._fhost, non_blocking=True)
                self._idev.copy_(self._ihost, non_blocking=True)
                fd, idv = self._fdev.view(6, -1), self._idev.view(3, -1)
                kw = dict(temperature=fd[0, :B], top_p=fd[1, :B], min_p=fd[2, :B], top_k=idv[0, :B].to(torch.int32),
                          seeds=idv[1, :B], steps=idv[2, :B].to(torch.int32))
                if any_pen:
                    counts = self._ensure_counts()
                    slot_rows = torch.tensor([s.request.slot for s in sched], dtype=torch.int64, device=self.device)
                    kw.update(presence=fd[3, :B], frequency=fd[4, :B], repetition=fd[5, :B],
                              counts=counts.index_select(0, slot_rows))
            tokens, _ = S.sample(logits, **kw)
            if any_pen:
                S.count_update(self.counts, tokens, torch.tensor([s.request.slot for s in sched], dtype=torch.int32,
                                                                  device=self.device))
        t3 = time.perf_counter()
        return tokens, t2, t3

    def _finish_launch(self, sched, B, tokens, t0, t1, t2, t3):
        # keep every slot's newest token on the device, and start the step's only device->host read
        self._last_tokens.index_copy_(0, self._dviews[7][:B].long(), tokens[:B].to(torch.int64))
        buf = self._tok_host[self._launches & 1]
        self._launches += 1
        event = None
        if self.device.type == "cuda":
            from ...ops import _lib

            self._tok_dev[:B].copy_(tokens[:B])
            self._tok_dev[B:B + 1].copy_(_lib.status_word(self.device)) if _lib.available() else \
                self._tok_dev[B:B + 1].zero_()
            buf[:B + 1].copy_(self._tok_dev[:B + 1], non_blocking=True)
            event = torch.cuda.Event()
            event.record()
        else:
            buf[:B].copy_(tokens[:B])
            buf[B] = 0
        tm = self.timings
        tm["prep"] += t1 - t0
        tm["exec"] += t2 - t1
        tm["sample"] += t3 - t2
        tm["steps"] += 1
        return (sched, B, buf, event)
