"""The engine: owns weights, paged KV, scheduler and the step loop.

``step()`` is the hot loop of the reference's ``InferenceRuntime::step``
(rust/engine/src/runtime.rs:2141-2150, :2212-3150): schedule -> build the ragged batch
-> forward -> sample / verify -> commit -> token events. Differences that matter on a
B200: per-step arrays travel in ONE pinned-host -> device copy; pure-decode steps
replay a captured CUDA graph per batch bucket (also inside a tensor-parallel group,
where the reference switches graphs off, docs/multi-gpu.md:94-96); greedy tokens are
picked on the device and only the ids come back.

Every rank of a tensor-parallel group runs this same class on the same request
stream (SPMD scheduling), so no step descriptor has to be broadcast; rank 0 is the
only one that reports events.
"""
from __future__ import annotations

import dataclasses
import os

import itertools
import time
from typing import Dict, Iterable, List, Optional, Sequence

import numpy as np
import torch

from ..config import EngineConfig, ModelConfig, ParallelConfig
from ..models.decoder import Decoder, KVCache, StepBatch
from ..models.weights import DecoderWeights, init_random_weights, make_shard_spec
from ..ops import get_ops
from .block_manager import BlockManager
from .request import Request, RequestStatus, SamplingParams, TokenEvent
from .scheduler import ScheduledSeq, ScheduledStep, Scheduler


class EngineStats:
    def __init__(self):
        self.steps = 0
        self.graph_steps = 0
        self.prefill_tokens = 0
        self.decode_tokens = 0
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self.schedule_ns = 0
        self.forward_calls = 0
        self.kernel_launches = 0
        self.spec_proposed = 0
        self.spec_accepted = 0


class LLMEngine:
    def __init__(self, model_cfg: ModelConfig, engine_cfg: Optional[EngineConfig] = None,
                 parallel: Optional[ParallelConfig] = None, device="cuda", weights: Optional[DecoderWeights] = None,
                 tp_group=None, tp_rank: int = 0, seed: int = 0, eos_token_id: Optional[int] = None,
                 ops=None, pp_group=None, stage: int = 0):
        self.model_cfg = model_cfg
        self.cfg = engine_cfg or EngineConfig()
        self.par = parallel or ParallelConfig()
        self.device = torch.device(device)
        self.is_cuda = self.device.type == "cuda"
        if self.is_cuda:
            torch.cuda.set_device(self.device)
        self.ops = ops or get_ops(self.device)
        self.tp_group, self.tp_rank = tp_group, tp_rank
        tp = self.par.tp
        self.spec = make_shard_spec(model_cfg, tp, tp_rank, self.par.expert_parallel)
        # pipeline stage: contiguous layer range, embedding on the first stage, head on the last
        self.pp_group, self.stage = pp_group, stage
        self.first_stage, self.last_stage = stage == 0, stage == self.par.pp - 1
        self.layer_range = self.par.stage_layers(model_cfg.num_layers, stage)
        self.weights = weights or init_random_weights(
            model_cfg, self.device, torch.bfloat16, seed, tp, tp_rank, self.par.expert_parallel,
            layers=self.layer_range, first_stage=self.first_stage, last_stage=self.last_stage)
        self.eos_token_id = eos_token_id
        if model_cfg.has_mla:
            # the latent pool has its own layout: the host / disk tiers, swapping and block export read the K / V pool
            if tp > 1:
                raise NotImplementedError("latent-attention layers are not cut over tensor-parallel ranks")
            self.cfg = dataclasses.replace(self.cfg, kv_tier_host_gb=0.0, kv_tier_disk_gb=0.0, preemption="recompute")
        if model_cfg.has_recurrent:
            # A recurrent state cannot be shared, rolled back or rebuilt from cached KV blocks: prompts are always
            # computed from their first token, rejected drafts would need a state snapshot per position, and a
            # preempted sequence is recomputed.
            if tp > 1:
                raise NotImplementedError("recurrent layers are not cut over tensor-parallel ranks")
            # With state checkpoints (state_cache_gb > 0) a prefix is reusable at the block boundaries where a copy
            # of the state was kept; without them prefix caching is off.
            keep_prefix = self.cfg.enable_prefix_caching and self.cfg.state_cache_gb > 0
            self.cfg = dataclasses.replace(self.cfg, enable_prefix_caching=keep_prefix, speculative="off", preemption="recompute",
                                           kv_tier_host_gb=0.0, kv_tier_disk_gb=0.0)
        self.block_size = self.cfg.block_size
        self.max_blocks_per_seq = -(-self.cfg.max_model_len // self.block_size)
        num_blocks = self.cfg.num_kv_blocks or self._size_kv_pool()
        if self.cfg.kv_cache_dtype not in ("bf16", "fp8", "fp8_e4m3", "fp32"):
            raise ValueError("kv_cache_dtype must be bf16 or fp8_e4m3")
        # fp32: only with the PyTorch operators (exact comparisons against other implementations on the CPU)
        kv_dtype = {"bf16": torch.bfloat16, "fp32": torch.float32}.get(self.cfg.kv_cache_dtype, torch.float8_e4m3fn)
        if kv_dtype == torch.float32 and hasattr(self.ops, "k"):
            raise ValueError("an fp32 KV pool is for the reference operators only")
        if model_cfg.has_mla:
            from ..models.mla import MlaCache
            if kv_dtype not in (torch.bfloat16, torch.float32):
                raise ValueError("the latent cache of multi-head latent attention is bf16")
            self.kv = MlaCache(self._kv_layers(), num_blocks, self.block_size,
                               model_cfg.mla["kv_lora_rank"] + model_cfg.mla["qk_rope_head_dim"], self.device, kv_dtype)
        else:
            self.kv = KVCache(self._kv_layers(), num_blocks, self.spec.hkv_local, self.block_size,
                              model_cfg.head_dim, self.device, kv_dtype)
        self.rstate = None
        if model_cfg.has_recurrent:
            # one state row per running sequence, a few spare for sequences between two owners, and the scratch
            # row that padding sequences of a captured step write to
            from ..models.recurrent import RecurrentState
            self.rstate = RecurrentState(model_cfg, self.layer_range, self.cfg.max_num_seqs + 9, self.device,
                                         self.weights.embed.dtype)
        self.decoder = Decoder(model_cfg, self.weights, self.kv, self.ops, self.spec, tp_group,
                               layer_range=self.layer_range, first_stage=self.first_stage,
                               last_stage=self.last_stage, rstate=self.rstate)
        # expert parallel with all-to-all dispatch: peer buffers for the rows each rank owns
        if (self.is_cuda and model_cfg.is_moe and self.par.expert_parallel and self.par.ep_dispatch == "alltoall"
                and tp > 1 and getattr(tp_group, "group", None) is not None):
            from ..comm.ep_a2a import EpAllToAll
            rows = -(-self.cfg.max_num_batched_tokens // tp)
            self.decoder.ep_a2a = EpAllToAll(tp, tp_rank, model_cfg.hidden_size, model_cfg.num_experts // tp, rows,
                                             model_cfg.experts_per_token, self.device, group=tp_group.group)
        self.blocks = BlockManager(num_blocks, self.block_size, self.cfg.enable_prefix_caching,
                                   self.cfg.watermark)
        if self.rstate is not None:
            self.blocks.enable_state_slots(self.rstate.slots - 1)
        window = model_cfg.sliding_window if (model_cfg.sliding_window and model_cfg.window_pattern is None) else 0
        self.scheduler = Scheduler(self.cfg, self.blocks, window)
        self.state_ckpt = None
        if self.rstate is not None and self.cfg.enable_prefix_caching:
            from .state_cache import StateCheckpoints
            self.state_ckpt = StateCheckpoints(self.rstate, int(self.cfg.state_cache_gb * (1 << 30)))
            self.blocks.state_has, self.blocks.state_restore = self.state_ckpt.has, self.state_ckpt.restore
            self.scheduler.chunk_align = self.block_size
        self.kv_tier = None
        disk_dir = self.cfg.kv_tier_disk_dir or os.environ.get("FLLM_KV_DISK_DIR")
        if self.cfg.enable_prefix_caching and (self.cfg.kv_tier_host_gb > 0 or (disk_dir and self.cfg.kv_tier_disk_gb > 0)):
            self._attach_kv_tier(disk_dir)
        if self.cfg.preemption == "swap":
            self.scheduler.swapper = _KvSwapper(self)
        self.requests: Dict[str, Request] = {}
        self._seq_ids = itertools.count()
        self._req_ids = itertools.count()
        self.stats = EngineStats()
        self.proposer = None                 # speculative drafts: NgramProposer / DraftModelProposer
        self.adaptive = None
        if self.cfg.speculative == "ngram":
            from .speculative import AdaptiveDraft, NgramProposer
            self.proposer = NgramProposer(self.cfg.draft_tokens)
            self.adaptive = AdaptiveDraft(self.cfg.draft_tokens)
        elif self.cfg.speculative == "suffix":
            from .speculative import AdaptiveDraft, SuffixProposer
            self.proposer = SuffixProposer(self.cfg.draft_tokens)
            # disk tier: $FLLM_SUFFIX_DIR/suffix-<model digest>.bin is read now and rewritten when the engine closes
            sdir = os.environ.get("FLLM_SUFFIX_DIR")
            if sdir:
                import hashlib
                self._suffix_digest = hashlib.blake2b(repr((model_cfg.name, model_cfg.vocab_size, model_cfg.hidden_size,
                                                            model_cfg.num_layers)).encode(), digest_size=16).digest()
                self._suffix_path = os.path.join(sdir, f"suffix-{self._suffix_digest.hex()}.bin")
                self.proposer.load(self._suffix_path, self._suffix_digest)
            self.adaptive = AdaptiveDraft(self.cfg.draft_tokens)
        self._graphs: Dict[int, "_DecodeGraph"] = {}
        self._graph_pool = None
        self._inflight = None                # launch-ahead: the decode step whose ids are still on the device
        # staging: [ids | positions | slots | row_seq | logit_rows | block tables]
        max_rows = max(self.cfg.max_num_seqs, self._bucket_for(self.cfg.max_num_seqs))
        cap = 5 * max(self.cfg.max_num_batched_tokens, max_rows) + max_rows * (self.max_blocks_per_seq + 3) + 64
        # one staging pair per pipeline micro-batch in flight (slot 0 is the only one without PP)
        self._stage_bufs = []
        for _ in range(max(1, self.par.pp)):
            hbuf = torch.empty(cap, dtype=torch.int32, pin_memory=self.is_cuda)
            self._stage_bufs.append((hbuf, hbuf.numpy(), torch.empty(cap, dtype=torch.int32, device=self.device)))
        self._host, self._host_np, self._dev = self._stage_bufs[0]
        # launch-ahead alternates two pinned host buffers (and two result buffers) over ONE device
        # staging buffer: the copy for step t+1 is queued behind step t's graph on the stream
        if self.par.pp == 1:
            halt = torch.empty(cap, dtype=torch.int32, pin_memory=self.is_cuda)
            self._stage_bufs.append((halt, halt.numpy(), self._dev))
        self._out_alt = torch.empty(512, dtype=torch.int32, pin_memory=self.is_cuda)
        self._flip = 0
        self._out_host = torch.empty(self.cfg.max_num_batched_tokens + 64, dtype=torch.int32,
                                     pin_memory=self.is_cuda)

    # ------------------------------------------------------------------ sizing
    def _kv_layers(self) -> int:
        """Attention layers of this stage (at least one, so that the pool tensors exist)."""
        return max(1, sum(1 for li in self.layer_range if self.model_cfg.has_kv(li)))

    def _size_kv_pool(self) -> int:
        per_block = KVCache.bytes_per_block(self._kv_layers(), self.spec.hkv_local,
                                            self.block_size, self.model_cfg.head_dim,
                                            2 if self.cfg.kv_cache_dtype == "bf16" else 1)
        if self.model_cfg.has_mla:
            from ..models.mla import MlaCache
            per_block = MlaCache.bytes_per_block(self._kv_layers(), self.block_size,
                                                 self.model_cfg.mla["kv_lora_rank"] + self.model_cfg.mla["qk_rope_head_dim"])
        if self.is_cuda:
            free, total = torch.cuda.mem_get_info(self.device)
            budget = int(total * self.cfg.gpu_memory_utilization) - (total - free)
            budget -= 4 << 30           # activations, graphs, workspaces
            if self.model_cfg.has_recurrent:
                from ..models.recurrent import RecurrentState
                budget -= RecurrentState.bytes_per_slot(self.model_cfg, self.layer_range) * (self.cfg.max_num_seqs + 9)
        else:
            budget = 256 << 20
        want = self.cfg.max_num_seqs * self.max_blocks_per_seq
        return max(64, min(budget // per_block, want))

    # ------------------------------------------------------------------ requests
    def add_request(self, prompt: Sequence[int], params: Optional[SamplingParams] = None,
                    request_id: Optional[str] = None, arrival: Optional[float] = None) -> str:
        params = params or SamplingParams()
        params.validate(self.model_cfg.vocab_size)
        prompt = [int(t) for t in prompt]
        if not prompt:
            raise ValueError("empty prompt")
        if len(prompt) + 1 > self.cfg.max_model_len:
            raise ValueError(f"prompt of {len(prompt)} tokens exceeds max_model_len={self.cfg.max_model_len}")
        rid = request_id or f"req-{next(self._req_ids)}"
        req = Request(rid, next(self._seq_ids), prompt, params)
        if arrival is not None:          # step control: every rank files the request under the leader's clock
            req.arrival = arrival
        self.requests[rid] = req
        self.scheduler.add(req)
        return rid

    def abort_request(self, request_id: str) -> bool:
        r = self.scheduler.abort(request_id)
        self.requests.pop(request_id, None)
        return r is not None

    def has_unfinished(self) -> bool:
        return self.scheduler.has_work() or self._inflight is not None

    # ------------------------------------------------------------------ disaggregated prefill / decode
    def export_request(self, request_id: str, remove: bool = True) -> dict:
        """Prefill side of disaggregated serving: the state of a request whose prompt has been
        processed (tokens, sampling parameters, and the KV blocks it owns, copied to the host), to be
        handed to ``import_request`` of another engine of the same model and KV layout
        (rust/engine/src/disagg.rs is the reference's KV hand-over)."""
        self.drain()
        r = self.requests.get(request_id)
        if r is None or r.finished:
            raise KeyError(f"no live request {request_id!r}")
        if not r.output or r.num_computed < len(r.prompt):
            raise ValueError("the prompt has not been processed yet")
        n = r.num_computed
        table = self.blocks.table(r.seq_id)[: self.blocks.blocks_needed(n)]
        live = [i for i, b in enumerate(table) if b >= 0]            # window-pruned blocks are not shipped
        idx = torch.tensor([table[i] for i in live], dtype=torch.long, device=self.device)
        kv = self.kv.store.index_select(2, idx).cpu() if live else self.kv.store[:, :, :0].cpu()
        import dataclasses
        params = {k: v for k, v in dataclasses.asdict(dataclasses.replace(r.params, guided=None)).items() if k != "guided"}
        blob = {"prompt": list(r.prompt), "output": list(r.output), "num_computed": n, "live_blocks": live,
                "kv": kv.view(torch.uint8) if kv.element_size() == 1 else kv, "kv_dtype": str(self.kv.store.dtype),
                "block_size": self.block_size, "params": params}
        if remove:
            self.scheduler.finish(r, "exported")
            self.requests.pop(request_id, None)
        return blob

    def import_request(self, blob: dict, request_id: Optional[str] = None) -> str:
        """Decode side: adopt an exported request. Its KV is copied into freshly allocated blocks and
        the request continues as a running decode sequence."""
        kv = blob["kv"]
        if blob["kv_dtype"] != str(self.kv.store.dtype) or blob["block_size"] != self.block_size:
            raise ValueError("KV layout mismatch between the exporting and the importing engine")
        if kv.element_size() == 1 and kv.dtype != self.kv.store.dtype:
            kv = kv.view(self.kv.store.dtype)
        want = self.kv.store.shape
        if tuple(kv.shape[:2]) != tuple(want[:2]) or tuple(kv.shape[3:]) != tuple(want[3:]):
            raise ValueError(f"KV shape {tuple(kv.shape)} does not fit this engine's pool {tuple(want)}")
        params = SamplingParams(**blob["params"])
        params.validate(self.model_cfg.vocab_size)
        n = int(blob["num_computed"])
        rid = request_id or f"req-{next(self._req_ids)}"
        req = Request(rid, next(self._seq_ids), [int(t) for t in blob["prompt"]], params)
        req.output = [int(t) for t in blob["output"]]
        req.num_computed = n
        self.blocks.allocate(req.seq_id, [])
        if not self.blocks.ensure_capacity(req.seq_id, n + 1):
            self.blocks.free_seq(req.seq_id)
            raise RuntimeError("not enough free KV blocks to import the request")
        table = self.blocks.table(req.seq_id)
        live = list(blob["live_blocks"])
        if live:
            dst = torch.tensor([table[i] for i in live], dtype=torch.long, device=self.device)
            self.kv.store.index_copy_(2, dst, kv.to(self.device))
        self.blocks.commit_tokens(req.seq_id, req.all_tokens, n, params.cache_salt.encode())
        req.status = RequestStatus.RUNNING
        self.scheduler.running.append(req)
        self.requests[rid] = req
        return rid

    def prefill_only(self, prompt: Sequence[int], params: Optional[SamplingParams] = None) -> "tuple[dict, list]":
        """Run a prompt until its first token exists and export it. Other requests keep being served
        by the same steps; their events are returned for the caller to deliver."""
        rid = self.add_request(prompt, params)
        events: List[TokenEvent] = []
        r = self.requests[rid]
        while not r.output and not r.finished:
            events.extend(self.step())
        events.extend(self.drain())
        if r.finished:
            raise RuntimeError(f"request finished during prefill: {r.finish_reason}")
        mine = [e for e in events if e.request_id == rid]
        return self.export_request(rid), [e for e in events if e.request_id != rid] if mine is not None else events

    # ------------------------------------------------------------------ batch building
    def _build_batch(self, step: ScheduledStep, pad_to: int = 0, slot: int = 0) -> StepBatch:
        seqs = step.seqs
        T = step.num_tokens
        B = len(seqs)
        Tp = max(T, pad_to)
        Bp = max(B, pad_to) if pad_to else B
        bs = self.block_size
        host_t, h, dev = self._stage_bufs[slot]
        ids = h[0:Tp]
        pos = h[Tp:2 * Tp]
        slots = h[2 * Tp:3 * Tp]
        rseq = h[3 * Tp:4 * Tp]
        rows: List[int] = []
        max_kv = 0
        max_blocks = 1
        for s in seqs:
            max_blocks = max(max_blocks, len(self.blocks.table(s.req.seq_id)))
        if pad_to:
            max_blocks = self.max_blocks_per_seq
        R_cap = Tp
        lrow = h[4 * Tp:4 * Tp + R_cap]
        o_qs, o_kl, o_tab = 5 * Tp, 5 * Tp + Bp + 1, 5 * Tp + 2 * Bp + 1
        qst = h[o_qs:o_qs + Bp + 1]
        kvl = h[o_kl:o_kl + Bp]
        tab = h[o_tab:o_tab + Bp * max_blocks].reshape(Bp, max_blocks)
        o_ss = o_tab + Bp * max_blocks
        sst = h[o_ss:o_ss + Bp] if self.rstate is not None else None
        max_q, min_q = 1, 1 << 30
        t = 0
        for i, s in enumerate(seqs):
            r = s.req
            n = s.count
            tb = self.blocks.np_table(r.seq_id)
            if n == 1 and not s.verify and r.output:       # decode row: no list building
                p0 = s.start
                ids[t] = r.output[-1] if p0 == r.num_tokens - 1 else r.all_tokens[p0]
                pos[t] = p0
                slots[t] = tb[p0 // bs] * bs + p0 % bs
            else:
                toks = r.prompt + r.output if not s.verify else r.prompt + r.output + r.draft
                ids[t:t + n] = toks[s.start:s.start + n]
                p = np.arange(s.start, s.start + n, dtype=np.int32)
                pos[t:t + n] = p
                slots[t:t + n] = tb[p // bs] * bs + p % bs
            rseq[t:t + n] = i
            tab[i, :tb.shape[0]] = tb
            qst[i] = t
            kvl[i] = s.start + n
            if sst is not None:
                sst[i] = self.blocks.state_slot(r.seq_id)
            max_q, min_q = max(max_q, n), min(min_q, n)
            if s.wants_logits:
                if s.verify:
                    rows.extend(range(t, t + n))
                else:
                    rows.append(t + n - 1)
            max_kv = max(max_kv, s.start + n)
            t += n
        if Tp > T:           # padding rows of a graph bucket: no KV write, row 0's table
            ids[T:Tp] = 0
            pos[T:Tp] = 0
            slots[T:Tp] = -1
            rseq[T:Tp] = 0
            rows.extend(range(T, Tp))
            qst[B:Bp] = np.arange(T, Tp, dtype=np.int32)      # one padding row per padding sequence
            kvl[B:Bp] = 1
            if sst is not None:
                sst[B:Bp] = self.rstate.slots - 1
            min_q = 1
        qst[Bp] = Tp
        R = len(rows)
        lrow[:R] = rows
        used = o_ss + (Bp if sst is not None else 0)
        if self.is_cuda:
            dev[:used].copy_(host_t[:used], non_blocking=True)
        else:
            dev[:used] = host_t[:used]
        self.stats.h2d_bytes += used * 4
        host_seqs = None
        if sst is not None and max_q >= 512 and not pad_to:
            # long prompt chunks of recurrent layers may take a matrix form that is set up from the host
            host_seqs = [(int(qst[i]), s.count, int(sst[i]), s.start == 0) for i, s in enumerate(seqs)]
        return StepBatch(
            host_seqs=host_seqs,
            token_ids=dev[0:Tp], positions=dev[Tp:2 * Tp], slots=dev[2 * Tp:3 * Tp],
            row_seq=dev[3 * Tp:4 * Tp], logit_rows=dev[4 * Tp:4 * Tp + R],
            block_tables=dev[o_tab:o_tab + Bp * max_blocks].view(Bp, max_blocks),
            q_starts=dev[o_qs:o_qs + Bp + 1], seq_lens=dev[o_kl:o_kl + Bp],
            seq_state=dev[o_ss:o_ss + Bp] if sst is not None else None,
            num_seqs=Bp, num_tokens=T, max_kv_len=max_kv, all_decode=step.all_decode,
            max_q_len=max_q, min_q_len=min(min_q, max_q))

    # ------------------------------------------------------------------ graphs
    def _bucket_for(self, n: int) -> int:
        for b in self.cfg.graph_buckets:
            if b >= n:
                return b
        return 0

    def _decode_with_graph(self, step: ScheduledStep) -> torch.Tensor:
        """Pure-decode step through a captured graph; returns greedy ids for the bucket rows."""
        n = len(step.seqs)
        bucket = self._bucket_for(n)
        g = self._graphs.get(bucket)
        if g is None:
            g = _DecodeGraph(self, bucket)
            self._graphs[bucket] = g
        batch = self._build_batch(step, pad_to=bucket)     # fills the static staging buffer
        g.replay()
        self.stats.graph_steps += 1
        return g.tokens, g.logits, batch

    # ------------------------------------------------------------------ step
    def enable_draft_model(self, draft_cfg, weights=None, k: Optional[int] = None, seed: int = 1) -> None:
        """Speculate with a small decoder (rust/engine/src/runtime.rs:1568 ``enable_draft``)."""
        from .speculative import AdaptiveDraft, DraftModelProposer
        if draft_cfg.vocab_size != self.model_cfg.vocab_size:
            raise ValueError("draft and target must share the vocabulary")
        self.proposer = DraftModelProposer(self, draft_cfg, k or self.cfg.draft_tokens, seed, weights)
        self.adaptive = AdaptiveDraft(k or self.cfg.draft_tokens)
        # the proposer marks how much of a sequence its own KV covers: stale after a recompute preemption,
        # garbage after an abort / expiry / finish
        self.scheduler.on_drop = lambda r: self.proposer.forget(r.seq_id)

    def _propose_drafts(self) -> None:
        # sampled verification reads the full logit rows, which a pipeline hands over as ids only
        modes = ("greedy", "sampled") if self.par.pp == 1 else ("greedy",)
        cands = [r for r in self.scheduler.running
                 if r.is_decode and not r.draft and r.params.spec_mode in modes]
        if not cands:
            return
        k = self.adaptive.length() if self.adaptive else self.cfg.draft_tokens
        ok = []
        for r in cands:
            room = min(k, r.params.max_tokens - len(r.output) - 1, self.cfg.max_model_len - r.num_tokens - 1)
            if room >= 1 and self.blocks.ensure_capacity(r.seq_id, r.num_tokens + room):
                ok.append((r, room))
        if not ok:
            return
        if hasattr(self.proposer, "propose_batch"):
            kk = min(room for _, room in ok)
            drafts = self.proposer.propose_batch([r for r, _ in ok], kk)
            for r, _ in ok:
                r.draft = drafts.get(r.seq_id, [])[:kk]
        else:
            for r, room in ok:
                r.draft = self.proposer.propose(r.all_tokens, room)[:room]
                r.draft_logits = None

    # ------------------------------------------------------------------ launch-ahead decode
    PLACEHOLDER = -1

    def _async_ok(self) -> bool:
        return (self.cfg.async_scheduling and self.is_cuda and self.cfg.use_cuda_graphs and self.par.pp == 1
                and hasattr(self.ops, "k")
                and self.proposer is None)

    def _graph_eligible(self, step: ScheduledStep) -> bool:
        # (the PyTorch reference operators read sizes back to the host, which a capture does not allow; the
        # expert-parallel all-to-all keeps its call number on the device, so it replays inside a graph)
        return (self.is_cuda and self.cfg.use_cuda_graphs and step.all_decode and self.par.pp == 1
                and hasattr(self.ops, "k")
                and not any(s.verify for s in step.seqs) and self._bucket_for(len(step.seqs)) > 0)

    def _precommit(self, fl) -> None:
        """Account for the in-flight step as if it had finished: every sequence advances by one
        token whose id is not known yet (a placeholder in its output)."""
        fl["slots"] = []
        for s in fl["step"].seqs:
            r = s.req
            if r.finished or r.status != RequestStatus.RUNNING:
                fl["slots"].append(-1)
                continue
            fl["slots"].append(len(r.output))
            self.scheduler.commit(s, [self.PLACEHOLDER], register=False)

    def _finalize(self, fl) -> List[TokenEvent]:
        """Read the in-flight step's ids, patch the placeholders, apply stop conditions."""
        fl["event"].synchronize()
        toks = fl["out"][: fl["n"]].tolist()
        self.stats.d2h_bytes += fl["n"] * 4
        events: List[TokenEvent] = []
        now = time.monotonic()
        for i, s in enumerate(fl["step"].seqs):
            r, slot = s.req, fl["slots"][i]
            if slot < 0 or r.finished or slot >= len(r.output):
                continue
            r.output[slot] = toks[i]
            # A request that schedule() preempted after this step was launched keeps its real token (it is in
            # the waiting queue, its blocks are gone): only a sequence that still owns blocks registers them.
            if r.status == RequestStatus.RUNNING and r.seq_id in self.blocks.seqs:
                self.blocks.commit_tokens(r.seq_id, r.all_tokens, r.num_computed, r.params.cache_salt.encode())
            self.stats.decode_tokens += 1
            if r.first_token_time is None:
                r.first_token_time = now
            r.last_token_time = now
            r.token_times.append(now)
            new = [toks[i]]
            reason = self._finish_reason(r, new)
            if reason:
                self.scheduler.finish(r, reason)
                self.requests.pop(r.request_id, None)
            if self.tp_rank == 0:
                events.append(TokenEvent(r.request_id, new, bool(reason), reason))
        self.stats.steps += 1
        return events

    def _launch_ahead(self, step: ScheduledStep, prev) -> dict:
        """Queue a decode step behind the in-flight one. Ids of rows that continue a placeholder
        are taken from the previous step's device-side result, never from the host."""
        n = len(step.seqs)
        bucket = self._bucket_for(n)
        g = self._graphs.get(bucket)
        if g is None:
            g = _DecodeGraph(self, bucket)
            self._graphs[bucket] = g
        self._flip ^= 1
        self._build_batch(step, pad_to=bucket, slot=0 if self._flip == 0 else len(self._stage_bufs) - 1)
        if prev is not None:
            prev_row = {s.req.seq_id: i for i, s in enumerate(prev["step"].seqs)}
            src = [prev_row.get(s.req.seq_id, -1) for s in step.seqs]
            need = [i for i, (s, j) in enumerate(zip(step.seqs, src))
                    if j >= 0 and s.req.output and s.req.output[-1] == self.PLACEHOLDER]
            if need:
                if len(need) == n and src == list(range(n)) and prev["graph"].tokens.shape[0] >= n:
                    self._dev[0:n].copy_(prev["tokens"][:n])
                else:
                    idx = torch.tensor([src[i] for i in need], dtype=torch.long, device=self.device)
                    dst = torch.tensor(need, dtype=torch.long, device=self.device)
                    self._dev[0:n].index_copy_(0, dst, prev["tokens"].index_select(0, idx))
        g.replay()
        self.stats.graph_steps += 1
        self.stats.forward_calls += 1
        self.stats.kernel_launches += g.launches
        # a private copy: the graph's static result is overwritten by the next replay
        toks_dev = g.tokens.clone()
        out = self._out_host if self._flip == 0 else self._out_alt
        out[:bucket].copy_(toks_dev, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        return {"step": step, "graph": g, "tokens": toks_dev, "out": out, "n": n, "event": ev, "slots": []}

    @torch.inference_mode()
    def step(self) -> List[TokenEvent]:
        if not self._async_ok():
            return self._step_sync()
        events: List[TokenEvent] = []
        prev = self._inflight
        if prev is not None:
            self._precommit(prev)
        t0 = time.perf_counter_ns()
        step = self.scheduler.schedule()
        self.stats.schedule_ns += time.perf_counter_ns() - t0
        for r in step.expired:
            events.append(TokenEvent(r.request_id, [], True, r.finish_reason, error=r.finish_reason))
            self.requests.pop(r.request_id, None)
        eligible = (not step.empty and self._graph_eligible(step) and not step.cow
                    and not any(s.req.params.needs_full_sampler for s in step.seqs))
        if eligible:
            nxt = self._launch_ahead(step, prev)
            if prev is not None:
                events.extend(self._finalize(prev))
            self._inflight = nxt
            return events
        # not a pure decode step: drain the pipeline, then run this step the ordinary way
        if prev is not None:
            events.extend(self._finalize(prev))
            self._inflight = None
            step.seqs = [s for s in step.seqs if not s.req.finished and s.req.status == RequestStatus.RUNNING]
        if not step.empty:
            events.extend(self._run_scheduled(step))
        return events

    def drain(self) -> List[TokenEvent]:
        """Wait for the launch-ahead step (if any) and commit it; returns its events."""
        fl = self._inflight
        if fl is None:
            return []
        self._precommit(fl)
        self._inflight = None
        return self._finalize(fl)

    @torch.inference_mode()
    def _step_sync(self) -> List[TokenEvent]:
        t0 = time.perf_counter_ns()
        if self.proposer is not None:
            self._propose_drafts()
        step = self.scheduler.schedule()
        self.stats.schedule_ns += time.perf_counter_ns() - t0
        events: List[TokenEvent] = []
        for r in step.expired:
            events.append(TokenEvent(r.request_id, [], True, r.finish_reason, error=r.finish_reason))
            self.requests.pop(r.request_id, None)
        if step.empty:
            return events
        events.extend(self._run_scheduled(step))
        return events

    def _run_scheduled(self, step: ScheduledStep) -> List[TokenEvent]:
        """Forward + sample + commit of one scheduled step, waiting for its result."""
        events: List[TokenEvent] = []
        for src, dst in step.cow:
            self.kv.store[:, :, dst].copy_(self.kv.store[:, :, src])
        use_graph = self._graph_eligible(step)
        l0 = getattr(self.ops, "launches", 0)
        if use_graph:
            tokens_dev, logits, batch = self._decode_with_graph(step)
            self.stats.kernel_launches += self._graphs[self._bucket_for(len(step.seqs))].launches
        elif self.par.pp > 1:
            tokens_dev = self._pipeline_forward(step)
        else:
            want_hidden = any(s.wants_logits and s.req.params.embed for s in step.seqs)
            if want_hidden and self.decoder.fused_tp:
                raise RuntimeError("embeddings are not available on the fused tensor-parallel path")
            self.decoder.capture_hidden = want_hidden
            batch = self._build_batch(step)
            logits = self.decoder.forward(batch)
            tokens_dev = self.decoder.greedy_tokens(logits)
            if want_hidden:
                self.decoder.capture_hidden = False
                hid = self.decoder.last_hidden.float().cpu()
                row = 0
                for s in step.seqs:
                    if not s.wants_logits:
                        continue
                    if s.req.params.embed:
                        s.req.embedding = hid[row].tolist()
                    row += s.count if s.verify else 1
        self.stats.forward_calls += 1
        needs_sampler = any(s.wants_logits and s.req.params.needs_full_sampler for s in step.seqs)
        if needs_sampler and self.par.pp == 1:
            tokens_dev = self._sample(step, logits, tokens_dev)
        verdicts = None
        if any(s.verify for s in step.seqs):
            verdicts = self._verify_drafts(step, logits if self.par.pp == 1 else None, tokens_dev)
        n_rows = tokens_dev.shape[0]
        out = self._out_host[:n_rows]
        out.copy_(tokens_dev, non_blocking=self.is_cuda)
        if self.is_cuda:
            torch.cuda.current_stream().synchronize()
        self.stats.d2h_bytes += n_rows * 4
        if verdicts is not None:
            step.verified = {}
            for idxs, res in verdicts:
                host = res.tolist()
                self.stats.d2h_bytes += res.numel() * 4
                for i, rec in zip(idxs, host):
                    step.verified[i] = (rec[0], rec[1:2 + rec[0]])
        self.stats.kernel_launches += getattr(self.ops, "launches", 0) - l0
        toks = out.tolist()
        events.extend(self._commit(step, toks))
        self.stats.steps += 1
        return events

    def _pp_recv_buffer(self, index: int, rows: int, hidden: int) -> torch.Tensor:
        """Receive buffer of micro-batch `index`: one per micro-batch in flight, grown on demand and kept."""
        bufs = self.__dict__.setdefault("_pp_recv_bufs", {})
        buf = bufs.get(index)
        if buf is None or buf.shape[0] < rows:
            buf = torch.empty(max(rows, 64), hidden, dtype=torch.bfloat16, device=self.device)
            bufs[index] = buf
        return buf[:rows]

    def _pipeline_forward(self, step: ScheduledStep) -> torch.Tensor:
        """One step over pipeline stages. The step is cut into micro-batches by sequence
        (rust/engine/src/parallel/decoder_shard.rs:313-341); every stage runs them in order, so
        stage s works on micro-batch i while stage s+1 works on i-1. The hand-over is the bf16
        residual stream [rows, hidden] sent device to device with the library's p2p, all receives of a step
        posted up front into per-micro-batch buffers so that transfer and compute overlap (the reference
        copies it through host memory, rust/engine/src/rust_decoder.rs:5900-5911). The last stage
        samples; the ids are broadcast so that every rank commits the same tokens."""
        from .scheduler import ScheduledStep as _Step
        pp, g = self.par.pp, self.pp_group
        n_mb = min(self.par.pipeline_microbatches or pp, len(step.seqs))
        per = -(-len(step.seqs) // n_mb)
        chunks = [step.seqs[i:i + per] for i in range(0, len(step.seqs), per)]
        subs = [_Step(seqs=c) for c in chunks]
        batches = [self._build_batch(sub, slot=i % len(self._stage_bufs)) if i < len(self._stage_bufs) else None
                   for i, sub in enumerate(subs)]
        H = self.model_cfg.hidden_size
        toks, pending = [], []
        # Every hand-over of the step is posted before the first layer runs, each into a buffer of its own: the
        # library's point-to-point stream then only waits for the sender, so micro-batch i + 1 crosses NVLink while
        # micro-batch i computes (posted one at a time, each receive would queue behind the previous compute).
        recvs = []
        if not self.first_stage:
            for i, sub in enumerate(subs):
                buf = self._pp_recv_buffer(i, sub.num_tokens, H)
                recvs.append((g.irecv(buf, self.stage - 1), buf))
        for i, sub in enumerate(subs):
            b = batches[i] if batches[i] is not None else self._build_batch(sub, slot=i % len(self._stage_bufs))
            x_in = None
            if not self.first_stage:
                w, x_in = recvs[i]
                w.wait()                                   # device-side wait on the NCCL path; host wait on gloo
            x, delta = self.decoder.forward_hidden(b, hidden_in=x_in)
            if not self.last_stage:
                out = (x.float() + delta.float()).to(x.dtype) if delta is not None else x
                pending.append((g.isend(out, self.stage + 1), out))
            else:
                lg = self.decoder.logits(x, delta, b)
                t = self.decoder.greedy_tokens(lg)
                if any(s.wants_logits and s.req.params.needs_full_sampler for s in sub.seqs):
                    t = self._sample(sub, lg, t)
                toks.append(t)
        for w, _ in pending:
            w.wait()
        n_rows = sum(len(range(s.count)) if s.verify else 1 for s in step.seqs if s.wants_logits)
        if self.last_stage:
            out = torch.cat(toks) if toks else torch.empty(0, dtype=torch.int32, device=self.device)
        else:
            out = torch.empty(n_rows, dtype=torch.int32, device=self.device)
        if n_rows:
            g.broadcast(out, src=pp - 1)
        return out

    SPEC_DRAW_BASE = 0x40000000              # keeps the acceptance draws apart from the sampler's own counter

    def _verify_drafts(self, step: ScheduledStep, logits: Optional[torch.Tensor], tokens_dev: torch.Tensor):
        """Acceptance of the step's drafts, decided on the device (rule: rust/engine/src/speculative.rs:103
        ``verify_chain``). Greedy requests compare draft ids with the target's argmax ids; sampled requests run
        the exact accept / residual rule on the logit rows, against the draft model's logits when the proposer
        kept them and against a point mass otherwise. Returns [(step.seqs indices, int32 [n, k + 2] on the
        device: accepted count, then the accepted drafts and the target's token)]; the caller reads it with
        the step's ids."""
        from .sampler import _row_params
        starts, row = {}, 0
        for i, s in enumerate(step.seqs):
            if s.wants_logits:
                starts[i] = row
                row += s.count if s.verify else 1
        out = []
        dev = tokens_dev.device
        for mode in ("greedy", "sampled"):
            grp = [i for i, s in enumerate(step.seqs) if s.verify and (s.req.params.spec_mode or "greedy") == mode]
            if not grp:
                continue
            if mode == "sampled" and logits is None:
                raise RuntimeError("sampled verification needs the logit rows of the step")
            k = max(step.seqs[i].verify for i in grp)
            meta = np.full((len(grp), k + 2), -1, dtype=np.int32)
            for j, i in enumerate(grp):
                s = step.seqs[i]
                assert starts[i] + s.verify + 1 <= row
                meta[j, :s.verify] = s.req.draft[:s.verify]
                meta[j, k], meta[j, k + 1] = s.verify, starts[i]
            m = torch.from_numpy(meta).to(dev)
            self.stats.h2d_bytes += meta.nbytes
            draft, nd, rs = m[:, :k].contiguous(), m[:, k].contiguous(), m[:, k + 1].contiguous()
            if mode == "greedy":
                n_acc, toks = self.ops.spec_verify_greedy(draft, tokens_dev.contiguous(), nd, rs)
            else:
                full = self.decoder.full_logits(logits)
                dls = [getattr(step.seqs[i].req, "draft_logits", None) for i in grp]
                dl = None
                if all(d is not None for d in dls):
                    V = full.shape[1]
                    dl = torch.zeros(len(grp), k, V, dtype=full.dtype, device=dev)
                    for j, d in enumerate(dls):
                        dl[j, :d.shape[0]] = d[:k].to(full.dtype)
                    dl = dl.view(len(grp) * k, V)
                params = []
                for i in grp:
                    r = step.seqs[i].req
                    params.append(_row_params(r, self.SPEC_DRAW_BASE + 2 * len(r.output), self.cfg.seed))
                n_acc, toks = self.ops.spec_verify_sampled(full, dl, draft, params, nd, rs)
            out.append((grp, torch.cat([n_acc.view(-1, 1), toks], 1)))
        return out

    def _sample(self, step: ScheduledStep, logits: torch.Tensor, greedy: torch.Tensor) -> torch.Tensor:
        from .sampler import sample_step
        full = self.decoder.full_logits(logits)
        return sample_step(self, step, full, greedy)

    def _commit(self, step: ScheduledStep, toks: List[int]) -> List[TokenEvent]:
        events: List[TokenEvent] = []
        now = time.monotonic()
        row = 0
        verified = getattr(step, "verified", None)
        for si, s in enumerate(step.seqs):
            r = s.req
            if not s.wants_logits:
                self.scheduler.commit(s, [])
                self.stats.prefill_tokens += s.count
                end = s.start + s.count
                if self.state_ckpt is not None and end % self.block_size == 0 and r.seq_id in self.blocks.seqs:
                    sb = self.blocks.seqs[r.seq_id]
                    if len(sb.hashes) >= end // self.block_size:       # the chunk's last block is registered: keep its state
                        self.state_ckpt.save(sb.hashes[end // self.block_size - 1], sb.state_slot)
                continue
            if s.verify:
                target = toks[row:row + s.count]
                row += s.count
                if verified is not None and si in verified:
                    acc, new = verified[si]
                    new = list(new)
                else:                                       # host statement of the greedy rule
                    acc = 0
                    while acc < s.verify and r.draft[acc] == target[acc]:
                        acc += 1
                    new = r.draft[:acc] + [target[acc]]
                r.draft_logits = None
                if self.adaptive is not None:
                    self.adaptive.update(s.verify, acc)
                self.stats.spec_proposed += s.verify
                self.stats.spec_accepted += acc
                self.scheduler.commit(s, new, accepted_drafts=acc)
            else:
                new = [toks[row]]
                row += 1
                self.scheduler.commit(s, new)
            if s.count > 1 and not s.verify:
                self.stats.prefill_tokens += s.count
            else:
                self.stats.decode_tokens += len(new)
            if r.params.guided is not None:
                for t in new:
                    r.params.guided.advance(t)
            if r.first_token_time is None:
                r.first_token_time = now
            r.last_token_time = now
            r.token_times.append(now)
            reason = self._finish_reason(r, new)
            if reason:
                # drop tokens generated past a stop inside a multi-token (speculative) commit
                self.scheduler.finish(r, reason)
                if hasattr(self.proposer, "forget"):
                    self.proposer.forget(r.seq_id)
                if hasattr(self.proposer, "observe"):
                    self.proposer.observe(r.prompt + r.output)       # the shared suffix index learns finished texts
                self.requests.pop(r.request_id, None)
            if self.tp_rank == 0:
                ev = TokenEvent(r.request_id, new, bool(reason), reason, embedding=getattr(r, "embedding", None))
                if r.params.logprobs and len(r.logprobs) >= len(new):
                    ev.logprobs = r.logprobs[-len(new):]
                    if r.params.top_logprobs > 0 and len(r.top_logprobs) >= len(new):
                        ev.top_logprobs = r.top_logprobs[-len(new):]
                events.append(ev)
        return events

    def _finish_reason(self, r: Request, new: List[int]) -> Optional[str]:
        p = r.params
        n_out = len(r.output)
        for i, t in enumerate(new):
            idx = n_out - len(new) + i + 1
            if idx < p.min_tokens:
                continue
            if (not p.ignore_eos and self.eos_token_id is not None and t == self.eos_token_id) \
                    or t in p.stop_token_ids:
                del r.output[idx:]
                del new[i + 1:]
                return "stop"
        if n_out >= p.max_tokens:
            del r.output[p.max_tokens:]
            return "length"
        if r.num_tokens >= self.cfg.max_model_len:
            return "length"
        return None

    # ------------------------------------------------------------------ scoring
    @torch.inference_mode()
    def token_logits(self, tokens: Sequence[int]) -> torch.Tensor:
        """Teacher-forced logits: row i is the fp32 distribution over the token after tokens[:i + 1]
        ([len(tokens), vocab], on the engine's device). The sequence is fed in chunks of at most
        ``max_num_batched_tokens`` rows whose logits are all kept (the batch shape a speculative verification
        uses); its KV blocks are freed afterwards. Single pipeline stage only."""
        if self.par.pp > 1:
            raise RuntimeError("token_logits needs a single pipeline stage")
        tokens = [int(t) for t in tokens]
        n = len(tokens)
        if n < 1:
            raise ValueError("no tokens")
        if n > self.cfg.max_model_len:
            raise ValueError(f"{n} tokens exceed max_model_len={self.cfg.max_model_len}")
        self.drain()
        req = Request("score-" + str(next(self._req_ids)), next(self._seq_ids), tokens[:1], SamplingParams(max_tokens=1))
        req.draft = tokens[1:]
        self.blocks.allocate(req.seq_id, [])
        out = []
        try:
            if not self.blocks.ensure_capacity(req.seq_id, n):
                raise RuntimeError("not enough free KV blocks for this sequence")
            step_max = self.cfg.max_num_batched_tokens
            off = 0
            while off < n:
                cnt = min(step_max, n - off)
                step = ScheduledStep(seqs=[ScheduledSeq(req, off, cnt, True, verify=cnt - 1)])
                batch = self._build_batch(step)
                logits = self.decoder.full_logits(self.decoder.forward(batch)).float()
                out.append(logits[-1:] if cnt == 1 else logits[:cnt])
                off += cnt
        finally:
            self.blocks.free_seq(req.seq_id)
        return torch.cat(out)

    def score_tokens(self, tokens: Sequence[int]) -> List[float]:
        """Log-probability of tokens[1:] given their prefixes (natural log): len(tokens) - 1 values.
        Perplexity = exp(-mean(score)) (the reference's ``ppl`` sub-command, rust/engine/src/ppl.rs)."""
        tokens = [int(t) for t in tokens]
        if len(tokens) < 2:
            return []
        lp = torch.log_softmax(self.token_logits(tokens)[:-1], -1)
        tgt = torch.tensor(tokens[1:], dtype=torch.long, device=lp.device)
        return lp.gather(1, tgt[:, None]).flatten().tolist()

    # ------------------------------------------------------------------ convenience
    def generate(self, prompts: Iterable[Sequence[int]], params: Optional[SamplingParams] = None) -> List[List[int]]:
        ids = [self.add_request(p, params) for p in prompts]
        outs: Dict[str, List[int]] = {i: [] for i in ids}
        while self.has_unfinished():
            for ev in self.step():
                if ev.request_id in outs:
                    outs[ev.request_id].extend(ev.token_ids)
        if self.tp_rank != 0:
            return []
        return [outs[i] for i in ids]

    def _attach_kv_tier(self, disk_dir: Optional[str]) -> None:
        """Evicted prefix-cache blocks go to host memory / disk under their chain hash and come back when a
        prompt reaches them again (runtime.kv_tier). Every tensor-parallel rank keeps its own shard."""
        from .kv_tier import KvTier
        st = self.kv.store                                   # [layers, 2, blocks, kv heads, block, head dim]
        block_bytes = st[:, :, 0].numel() * st.element_size()
        # The signature names the model AND its weights: two checkpoints (or two random seeds) of one
        # architecture must never re-use each other's KV files. A directory belongs to one model.
        mc = self.model_cfg
        probe = [self.weights.final_norm]
        if self.weights.layers:
            l0 = self.weights.layers[0]
            probe += [t for t in (l0.attn_norm, l0.wqkv if isinstance(l0.wqkv, torch.Tensor) else None) if t is not None]
        import hashlib
        fp = hashlib.sha256()
        for t in probe:
            fp.update(t.detach().reshape(-1)[:4096].float().cpu().numpy().tobytes())
        sig = (f"{mc.name}|{tuple(st[:, :, 0].shape)}|{st.dtype}|bs{self.block_size}|tp{self.tp_rank}|"
               f"theta{mc.rope_theta}|{mc.rope_scaling.kind}:{mc.rope_scaling.factor}|w{fp.hexdigest()[:16]}")
        if self.tp_group is not None and getattr(self.tp_group, "size", 1) > 1:
            # ranks must take identical hit / miss decisions to keep their block tables equal: the host tier is
            # deterministic, a file that fails to read on one rank is not, so the disk tier is single-rank only
            disk_dir = None
        self.kv_tier = KvTier(sig, block_bytes, int(self.cfg.kv_tier_host_gb * (1 << 30)), disk_dir,
                              int(self.cfg.kv_tier_disk_gb * (1 << 30)))

        def evict(block: int, h: bytes) -> None:
            self.kv_tier.put(h, st[:, :, block].contiguous().view(torch.uint8).reshape(-1).cpu())

        def restore(h: bytes, block: int) -> bool:
            blob = self.kv_tier.get(h)
            if blob is None:
                return False
            st[:, :, block].copy_(blob.view(st.dtype).view(st[:, :, block].shape).to(st.device))
            return True
        self.blocks.on_evict, self.blocks.tier_has, self.blocks.tier_restore = evict, self.kv_tier.has, restore

    def beam_search(self, prompt: Sequence[int], beam_width: int = 4, max_tokens: int = 32, length_penalty: float = 1.0,
                    eos_token_id: Optional[int] = None, early_stopping: bool = True,
                    other_events: Optional[list] = None) -> "List[tuple]":
        """Beam search over this engine: -> [(tokens, score)] best first, score = sum of log-probabilities divided
        by len(tokens) ** length_penalty. Every round submits one one-token request per live beam that asks for
        its 2 x beam_width best continuations; the beams of a round run as one batch, and the prefix cache makes a
        beam's request re-use its parent's full KV blocks, so a round computes at most one block per beam
        Events of other requests that advance while the search steps the engine are appended to
        `other_events` (rust/engine/src/beam.rs is the reference's beam search)."""
        if not 1 <= beam_width <= 10:
            raise ValueError("beam_width must be in [1, 10]")
        eos = eos_token_id if eos_token_id is not None else self.eos_token_id
        prompt = [int(t) for t in prompt]
        norm = lambda toks, lp: lp / (max(len(toks), 1) ** length_penalty)
        live: "List[tuple]" = [([], 0.0)]
        done: "List[tuple]" = []
        room = self.cfg.max_model_len - len(prompt) - 1
        for _ in range(max(0, min(max_tokens, room))):
            reqs = []
            for toks, lp in live:
                sp = SamplingParams(max_tokens=1, temperature=0.0, logprobs=True, top_logprobs=2 * beam_width, ignore_eos=True)
                reqs.append((self.requests[self.add_request(prompt + toks, sp)], toks, lp))
            mine = {r.request_id for r, _, _ in reqs}
            while any(not r.finished for r, _, _ in reqs):
                for ev in self.step():
                    if other_events is not None and ev.request_id not in mine:
                        other_events.append(ev)
            # every tensor-parallel rank samples from the same gathered logits, so all ranks build the same beams
            cands = []
            for r, toks, lp in reqs:
                for t, l in (r.top_logprobs[0] if r.top_logprobs else []):
                    cands.append((toks + [int(t)], lp + float(l)))
            cands.sort(key=lambda c: -c[1])
            live = []
            for toks, lp in cands:
                if eos is not None and toks[-1] == eos:
                    if len(live) < beam_width:          # an ended hypothesis only counts while it ranks among the beams
                        done.append((toks, lp))
                elif len(live) < beam_width:
                    live.append((toks, lp))
                if len(live) >= beam_width:
                    break
            if not live:
                break
            if early_stopping and len(done) >= beam_width:
                worst_done = sorted(norm(t, l) for t, l in done)[-beam_width]
                # log-probabilities only fall: with a length penalty <= 1 no live beam can still overtake
                if length_penalty <= 1.0 and max(norm(t, l) for t, l in live) <= worst_done:
                    break
        if self.tp_rank != 0:
            return []
        final = done + live
        final.sort(key=lambda c: -norm(c[0], c[1]))
        return [(t, norm(t, l)) for t, l in final[:beam_width]]

    def close(self) -> None:
        """Drop captured graphs (they pin the library communicator: it cannot be destroyed while a
        graph that captured one of its collectives is alive) and wait for the device."""
        if getattr(self, "_suffix_path", None) and self.tp_rank == 0 and self.stage == 0:
            try:
                os.makedirs(os.path.dirname(self._suffix_path), exist_ok=True)
                self.proposer.save(self._suffix_path, self._suffix_digest)
            except OSError:
                pass                      # the tier is an optimisation: a full or read-only disk must not fail a shutdown
        self._graphs.clear()
        self._graph_pool = None
        import gc
        gc.collect()
        if self.is_cuda:
            torch.cuda.synchronize(self.device)

    def warm_up(self, buckets: Optional[Sequence[int]] = None) -> None:
        """Capture decode graphs ahead of traffic (rust/engine/src/runtime.rs:1085-1175)."""
        if not (self.is_cuda and self.cfg.use_cuda_graphs):
            return
        for b in buckets or self.cfg.graph_buckets:
            if b <= self.cfg.max_num_seqs and b not in self._graphs:
                self._graphs[b] = _DecodeGraph(self, b)
        self.settle_host()

    @staticmethod
    def settle_host() -> None:
        """Move everything allocated so far (weights, graphs, modules) out of the garbage collector's
        young generations. A full collection over a loaded engine walks millions of objects and showed
        up as 40 - 60 ms stalls of single decode steps at deterministic step numbers."""
        import gc
        gc.collect()
        gc.freeze()


class _KvSwapper:
    """Host tier for preempted requests: a victim's KV blocks are copied to (pinned) host memory instead of
    being recomputed later, and copied back into fresh blocks when it is scheduled again. Copies are
    ordered on the compute stream, after any step still in flight that writes those blocks."""

    def __init__(self, eng: "LLMEngine"):
        self.eng = eng
        self.parked: Dict[int, "tuple[torch.Tensor, List[int]]"] = {}
        self.bytes = 0
        self.limit = int(eng.cfg.swap_space_gb * (1 << 30))
        self.stats = {"swapped_out": 0, "swapped_in": 0, "refused": 0}

    def swap_out(self, req) -> bool:
        eng = self.eng
        n = req.num_computed
        table = eng.blocks.table(req.seq_id)[: eng.blocks.blocks_needed(n)]
        live = [i for i, b in enumerate(table) if b >= 0]
        per_block = eng.kv.store[:, :, 0].numel() * eng.kv.store.element_size()
        if self.bytes + len(live) * per_block > self.limit:
            self.stats["refused"] += 1
            return False
        idx = torch.tensor([table[i] for i in live], dtype=torch.long, device=eng.device)
        host = eng.kv.store.index_select(2, idx).cpu() if live else eng.kv.store[:, :, :0].cpu()
        self.parked[req.seq_id] = (host, live)
        self.bytes += host.numel() * host.element_size()
        self.stats["swapped_out"] += 1
        return True

    def swap_in(self, req) -> None:
        eng = self.eng
        host, live = self.parked.pop(req.seq_id)
        self.bytes -= host.numel() * host.element_size()
        table = eng.blocks.table(req.seq_id)
        if live:
            dst = torch.tensor([table[i] for i in live], dtype=torch.long, device=eng.device)
            eng.kv.store.index_copy_(2, dst, host.to(eng.device, non_blocking=False))
        self.stats["swapped_in"] += 1

    def drop(self, req) -> None:
        ent = self.parked.pop(req.seq_id, None)
        if ent is not None:
            self.bytes -= ent[0].numel() * ent[0].element_size()


class _DecodeGraph:
    """One captured decode step for a fixed number of rows. Inputs are read from the engine's
    device staging buffer at the fixed offsets `_build_batch(pad_to=bucket)` uses."""

    def __init__(self, eng: LLMEngine, bucket: int):
        self.bucket = bucket
        dev = eng._dev
        n, mb = bucket, eng.max_blocks_per_seq
        o_qs, o_kl, o_tab = 5 * n, 6 * n + 1, 7 * n + 1
        self.batch = StepBatch(
            token_ids=dev[0:n], positions=dev[n:2 * n], slots=dev[2 * n:3 * n], row_seq=dev[3 * n:4 * n],
            logit_rows=dev[4 * n:5 * n], block_tables=dev[o_tab:o_tab + n * mb].view(n, mb),
            q_starts=dev[o_qs:o_qs + n + 1], seq_lens=dev[o_kl:o_kl + n],
            seq_state=dev[o_tab + n * mb:o_tab + n * mb + n] if eng.rstate is not None else None,
            num_seqs=n, num_tokens=n, max_kv_len=eng.cfg.max_model_len, all_decode=True,
            max_q_len=1, min_q_len=1)
        # harmless contents for warm-up / capture: all rows padded
        dev[0:2 * n].zero_()
        dev[2 * n:3 * n].fill_(-1)
        dev[3 * n:4 * n].zero_()
        dev[4 * n:5 * n].copy_(torch.arange(n, dtype=torch.int32, device=dev.device))
        dev[o_qs:o_qs + n + 1].copy_(torch.arange(n + 1, dtype=torch.int32, device=dev.device))
        dev[o_kl:o_kl + n].fill_(1)
        dev[o_tab:o_tab + n * mb].zero_()
        if eng.rstate is not None:           # warm-up and capture write the scratch row only
            dev[o_tab + n * mb:o_tab + n * mb + n].fill_(eng.rstate.slots - 1)
        stream = torch.cuda.Stream(device=eng.device)
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            for _ in range(2):
                lg = eng.decoder.forward(self.batch)
                eng.decoder.greedy_tokens(lg)
        torch.cuda.current_stream().wait_stream(stream)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        if eng._graph_pool is None:
            eng._graph_pool = torch.cuda.graph_pool_handle()
        l0 = getattr(eng.ops, "launches", 0)
        with torch.cuda.graph(self.graph, pool=eng._graph_pool):
            self.logits = eng.decoder.forward(self.batch)
            self.tokens = eng.decoder.greedy_tokens(self.logits)
        self.launches = getattr(eng.ops, "launches", 0) - l0     # kernels replayed per step

    def replay(self) -> None:
        self.graph.replay()
