"""Worker runtime: one ModelRunner per GPU (or per CPU rank in tests).

Owns the model shard, the KV cache, input preparation, CUDA-graph replay for decode, sampling and the
host<->device block swap.  All traffic with the controller is bytes of the native wire format.

Parity: reference runtime/runner/model_runner.py:223 (ModelRunner) - dist init :351-559, allocate_kvcache
:685-917, run_model :1539-1621 (eager for prefill, graphs for decode), _standard_sample :1743-1826,
prepare_from_bytes :1829-1948, run_prepared :1984-2132, step timers :84-197; runtime/runner/input_preparer.py:36-393.
"""
from __future__ import annotations

import os
import time
from typing import Dict, List, Optional

import numpy as np
import torch
import torch.distributed as dist

from .._native import _core as C
from ..config import Config
from ..models.registry import get_model_class
from ..models.weights import expert_owner_filter, iterate_safetensors, random_hf_weights
from ..parallel.dist import DistContext, ParallelSpec, get_dist_context, init_dist_context
from .cache import KVCache, kv_budget_blocks, make_cache_plan, torch_dtype
from .context import ForwardContext
from .sampler import Sampler
from ..utils import nvtx


class StepTimer:
    """CPU phase timer plus optional CUDA-event forward timing (enabled by Config.step_timing)."""

    def __init__(self, enabled: bool, cuda: bool):
        self.enabled, self.cuda = enabled, cuda
        self.phases: Dict[str, float] = {}
        self._t0 = None
        self._ev = None
        self.last_forward_ms = 0.0

    def start(self, name):
        if self.enabled:
            self._t0 = (name, time.perf_counter())

    def stop(self):
        if self.enabled and self._t0:
            n, t = self._t0
            self.phases[n] = self.phases.get(n, 0.0) + (time.perf_counter() - t) * 1e3
            self._t0 = None

    def forward_begin(self):
        if self.enabled and self.cuda:
            self._ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            self._ev[0].record()

    def forward_end(self):
        if self.enabled and self.cuda and self._ev:
            self._ev[1].record()
            self._ev[1].synchronize()
            self.last_forward_ms = self._ev[0].elapsed_time(self._ev[1])


class ModelRunner:
    def __init__(self, config: Config, rank: int = 0, world_size: int = 1, device: Optional[str] = None,
                 dist_ctx: Optional[DistContext] = None):
        self.config = config
        self.rank, self.world_size = rank, world_size
        if device is None:
            use_cuda = config.device == "cuda" or (config.device == "auto" and torch.cuda.is_available())
            device = f"cuda:{int(os.environ.get('LOCAL_RANK', rank)) % max(1, torch.cuda.device_count())}" if use_cuda else "cpu"
        self.device = torch.device(device)
        if self.device.type == "cuda":
            torch.cuda.set_device(self.device)
        self.dtype = torch_dtype(config.dtype)
        self.dist = dist_ctx or init_dist_context(config.parallel_spec(), rank, world_size, self.device)
        self.mc = config.model_config
        self.model = None
        self.mtp = None
        self.cache: Optional[KVCache] = None
        self.sampler = Sampler(config.seed + 1000 * self.dist.attn_dp_rank, self.device)
        self.timer = StepTimer(config.step_timing, self.device.type == "cuda")
        self.graphs = None
        self.mtp_runner = None
        self._profiler = None
        self.h2d_bytes = 0          # bytes copied host -> device for step inputs (benchmark bookkeeping)
        self.d2h_bytes = 0          # bytes read back (sampled tokens, log-probabilities)
        self._last_decode = None
        self.plan = make_cache_plan(self.mc, config.resolved_kv_dtype(), config.kvcache_block_size, config.attention_tp,
                                    num_mtp_layers=self._num_mtp_layers(), use_indexer=config.use_nsa(), state_slots=config.max_num_seqs,
                                    hisparse_rows=config.hisparse_device_buffer_size if config.enable_hisparse else 0,
                                    max_ctx=(config.max_model_len or self.mc.max_position_embeddings))

    def _num_mtp_layers(self) -> int:
        return max(1, self.mc.num_nextn_predict_layers) if self.config.num_speculative_tokens > 0 else 0

    # ---- model -------------------------------------------------------------------------------
    def layer_range(self):
        L, pp = self.mc.num_hidden_layers, self.config.pp
        if pp == 1:
            return (0, L)
        from ..models.pp import pp_layer_partition
        return pp_layer_partition(L, pp)[self.dist.pp_rank]

    def init_model(self) -> None:
        cls = get_model_class(self.mc.architecture)
        if self.mc.quant == "fp8":
            # before any weight is quantised or loaded: the quantisers and the block-scaled GEMMs follow this setting
            from .. import ops
            (ops._get_sm100() if self.device.type == "cuda" else ops.reference).set_scale_format(self.config.resolved_scale_format())
        from ..parallel.ep import set_routing_options
        set_routing_options(balance_ranks=self.dist.ep_size if self.config.dummy_eplb else 0)
        from ..parallel import eplb
        plan = None
        if self.config.eplb_redundant_experts > 0:
            rows = self.mc.num_hidden_layers + max(1, self.mc.num_nextn_predict_layers)
            if self.config.eplb_load_path:
                load = torch.load(self.config.eplb_load_path, map_location="cpu").float()
                if load.shape[0] < rows:                       # layers the measurement does not cover (MTP blocks): uniform
                    load = torch.cat([load, torch.ones(rows - load.shape[0], load.shape[1])], 0)
            else:
                load = torch.ones(rows, self.mc.n_routed_experts)
            plan = eplb.EplbPlan.from_load(load, self.config.eplb_redundant_experts, self.dist.ep_size, 1)
        eplb.set_active_plan(plan)
        torch.manual_seed(self.config.seed)
        lr = self.layer_range()
        self.model = cls(self.mc, dtype=self.dtype, device=self.device, layer_range=lr if self.config.pp > 1 else None)
        keep = expert_owner_filter(self.mc, self.dist.ep_size, self.dist.ep_rank, lr if self.config.pp > 1 else None)
        want_mtp = self.config.num_speculative_tokens > 0
        if want_mtp:
            from ..models.deepseek import DeepseekMTP
            self.mtp = DeepseekMTP(self.mc, self.dtype, self.device, self.model.model.embed_tokens, self.model.lm_head)
        if self.config.dummy_weight:
            it = random_hf_weights(self.mc, self.config.seed, self.device, keep, include_mtp=want_mtp)
        else:
            it = iterate_safetensors(self.config.model, keep, self.device)
        self.load_weights(it)
        self.model.eval()
        if self.device.type == "cuda" and self.dist.ep_size > 1:
            from ..parallel import fused_moe
            fused_moe.install(self.config, self.dist)
        if self.device.type == "cuda" and self.dist.attn_tp_size > 1:
            from ..parallel import fused_tp
            fused_tp.install(self.config, self.dist, "attn_tp")

    def load_weights(self, it) -> int:
        if self.mtp is not None:
            from ..models.weights import load_deepseek_weights
            return load_deepseek_weights(self.model, it, mtp=self.mtp)
        return self.model.load_weights(it)

    def update_weights(self, src) -> int:
        """Replace the weights in place from a checkpoint directory or an iterable of (name, tensor).  Copies derived from a
        weight (the K-major forms of the absorbed MLA matrices) are rebuilt by the modules that own them, and the decode
        graphs, which captured the old copies' addresses, are re-created."""
        keep = expert_owner_filter(self.mc, self.dist.ep_size, self.dist.ep_rank, None)
        it = iterate_safetensors(src, keep, self.device) if isinstance(src, str) else ((n, t) for n, t in src if keep(n))
        n = self.load_weights(it)
        self._after_weight_change()
        return n

    def _after_weight_change(self) -> None:
        for m in list(self.model.modules()) + (list(self.mtp.modules()) if self.mtp is not None else []):
            if hasattr(m, "refresh_absorbed"):
                m.refresh_absorbed()
        if getattr(self, "l3", None) is not None:
            self.l3.bump_generation()            # blocks on disk were computed with the old weights
        if self.device.type == "cuda" and self.graphs is not None:
            self.graphs = type(self.graphs)(self)
            if self.has_collectives():
                self.graphs.capture_all()

    def export_weights(self, direct: bool = False) -> Dict[str, object]:
        """Descriptors of every parameter and buffer of this worker's shard, from which a worker process on the same machine
        (a serving replica with the same parallel layout and rank) can map the tensors and copy them over NVLink.  `direct`:
        the tensors themselves, for a replica in this process.
        Parity: reference runtime/context/parameter.py:91-140 (named regions registered for one-sided weight reads)."""
        from ..parallel.kv_transfer import export_tensor
        out = {}
        mods = [("", self.model)] + ([("mtp.", self.mtp)] if self.mtp is not None else [])
        for prefix, mod in mods:
            for n, p in list(mod.named_parameters()) + list(mod.named_buffers()):
                t = p.detach()
                if direct or not t.is_cuda:
                    out[prefix + n] = t
                else:
                    flat = (t.view(torch.uint8) if t.dtype == torch.float8_e4m3fn else t).contiguous().view(-1).view(torch.uint8)
                    assert flat.data_ptr() == t.data_ptr(), f"{n}: parameters must be contiguous to be exported"
                    out[prefix + n] = {"desc": export_tensor(flat, False), "dtype": str(t.dtype), "shape": list(t.shape)}
        return out

    def pull_weights(self, peer: Dict[str, object]) -> int:
        """Copy every tensor of `peer` (another worker's `export_weights()`) into this worker's parameters in place - one
        device-to-device copy per tensor, over NVLink when the peer sits on another GPU - then rebuild what is derived from
        the weights.  Names and shapes must match (same model, same parallel layout, same rank).
        Parity: reference runtime/context/parameter.py:169-228 (pull + in-place apply), engine/weight_sync.py."""
        from ..parallel.kv_transfer import open_tensor
        mine = {}
        mods = [("", self.model)] + ([("mtp.", self.mtp)] if self.mtp is not None else [])
        for prefix, mod in mods:
            for n, p in list(mod.named_parameters()) + list(mod.named_buffers()):
                mine[prefix + n] = p
        missing = sorted(set(mine) - set(peer))
        if missing:
            raise ValueError(f"the peer does not hold {len(missing)} of this worker's tensors, e.g. {missing[:3]}")
        n = 0
        with torch.no_grad():
            for name, dst in mine.items():
                src = peer[name]
                if isinstance(src, dict):
                    if list(dst.shape) != src["shape"] or str(dst.dtype) != src["dtype"]:
                        raise ValueError(f"{name}: peer has {src['dtype']} {src['shape']}, this worker {dst.dtype} {list(dst.shape)}")
                    raw = open_tensor(src["desc"])
                    d8 = (dst.view(torch.uint8) if dst.dtype == torch.float8_e4m3fn else dst).view(-1).view(torch.uint8)
                    d8.copy_(raw, non_blocking=True)
                else:
                    if dst.shape != src.shape or dst.dtype != src.dtype:
                        raise ValueError(f"{name}: peer has {src.dtype} {list(src.shape)}, this worker {dst.dtype} {list(dst.shape)}")
                    dst.copy_(src, non_blocking=True)
                n += 1
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        self._after_weight_change()
        return n

    # ---- cache -------------------------------------------------------------------------------
    def profile_num_blocks(self) -> int:
        """How many KV blocks fit: run a worst-case prefill to find peak activation memory, then apply the budget formula."""
        if self.config.num_kvcache_blocks is not None:
            return self.config.num_kvcache_blocks
        if self.device.type != "cuda":
            return 256
        torch.cuda.synchronize()
        torch.cuda.reset_peak_memory_stats()
        free, total = torch.cuda.mem_get_info()
        current = torch.cuda.memory_allocated()
        # activation peak estimate from a synthetic prefill of the configured token budget
        try:
            self._warmup_prefill(min(self.config.max_num_batched_tokens, 8192))
        finally:
            torch.cuda.synchronize()
        peak = torch.cuda.max_memory_allocated()
        used = total - free
        torch.cuda.empty_cache()
        blocks = kv_budget_blocks(self.plan, total, self.config.gpu_memory_utilization, used, peak, current,
                                  reserved=self.plan.state_bytes + self.plan.hisparse_device_bytes)
        if self.plan.hisparse:      # the cold tier is bounded by the pinned host memory it may take
            blocks = min(blocks, int(self.config.hisparse_host_gb * (1 << 30)) // max(1, self.plan.kv_block_bytes))
        return blocks

    def _warmup_prefill(self, tokens: int) -> None:
        bs = self.plan.block_size
        nb = (tokens + bs - 1) // bs
        import dataclasses
        tmp = KVCache(dataclasses.replace(self.plan, state_slots=0), nb, self.device)   # the scratch state slot is enough here
        b = C.RunnerIn()
        b.is_prefill = True
        b.seq_ids = [0]
        b.input_ids = [1] * tokens
        b.positions = list(range(tokens))
        b.q_lens, b.seq_lens = [tokens], [tokens]
        b.block_tables, b.block_offsets = list(range(nb)), [0, nb]
        b.temperatures, b.sample_mask = [0.0], [1]
        b.state_slots = b.handoff_slots = b.hisparse_slots = [-1]
        saved, self.cache = self.cache, tmp
        try:
            self.run_batch(b)
        finally:
            self.cache = saved
            del tmp

    def allocate_kvcache(self, num_blocks: int) -> None:
        self.cache = KVCache(self.plan, num_blocks, self.device)
        if self.device.type == "cuda":
            from ..ops import sm100
            rows = (num_blocks + 1) * self.plan.block_size
            if self.plan.hisparse:                      # the key path writes into the hot buffers there
                rows = max(rows, (self.plan.hs_slots + 1) * self.plan.hot_rows)
            sm100.debug_set_bounds(rows, num_blocks + 1, self.plan.state_slots + 1 if self.plan.gdn else 0, self.mc.n_routed_experts)
        self.cache.allocate_host(self.config.num_host_kvcache_blocks)
        if self.config.num_speculative_tokens > 0:
            from .mtp_runner import MTPRunner
            self.mtp_runner = MTPRunner(self)
        from ..parallel.ep import get_fused_backend
        # the NCCL all-gather EP path sizes its buffers from a host read-back and cannot be captured; the fused path can
        ep_capturable = self.dist.ep_size == 1 or get_fused_backend() is not None
        if self.device.type == "cuda" and not self.config.enforce_eager and ep_capturable:
            from .graph_runner import DecodeGraphRunner
            self.graphs = DecodeGraphRunner(self)
            if self.mtp_runner is not None:
                from .mtp_runner import MTPGraphRunner
                self.mtp_runner.graphs = MTPGraphRunner(self, self.mtp_runner)
            if self.has_collectives():
                self.graphs.capture_all()
                if self.mtp_runner is not None:
                    self.mtp_runner.graphs.capture_all()

    def has_collectives(self) -> bool:
        """True when a forward pass talks to other ranks (expert- or tensor-parallel groups), i.e. when every rank has to run
        the same sequence of forward passes."""
        return self.dist.ep_size > 1 or self.dist.attn_tp_size > 1

    # ---- input preparation ---------------------------------------------------------------------
    def _to_dev(self, arr: np.ndarray, dtype=None) -> torch.Tensor:
        t = torch.from_numpy(arr)
        if dtype is not None:
            t = t.to(dtype)
        if self.device.type == "cuda":
            self.h2d_bytes += t.numel() * t.element_size()
            return t.pin_memory().to(self.device, non_blocking=True)
        return t

    def prepare(self, b) -> ForwardContext:
        bs = self.plan.block_size
        if b.is_dummy or b.num_seqs == 0:
            return self._dummy_context(b.is_prefill)
        d = b.prepare(bs, 0)
        q_lens = b.q_lens
        uniform = q_lens[0] if all(q == q_lens[0] for q in q_lens) else 0
        ctx = ForwardContext(
            is_prefill=b.is_prefill, num_seqs=b.num_seqs, num_tokens=len(b.input_ids),
            cu_seqlens_q=self._to_dev(d["cu_seqlens_q"]), context_lens=self._to_dev(d["context_lens"]),
            slot_mapping=self._to_dev(d["slot_mapping"]), block_tables=self._to_dev(d["block_tables"]).view(b.num_seqs, -1),
            max_seqlen_q=int(d["max_seqlen_q"]), max_seqlen_k=int(d["max_seqlen_k"]),
            last_token_indices=self._to_dev(d["last_token_indices"]), q_len_uniform=uniform,
            kv_caches=self.cache.layers, indexer_caches=self.cache.indexer_layers,
            cu_seqlens_q_host=d["cu_seqlens_q"].tolist(), context_lens_host=d["context_lens"].tolist())
        ctx.extras["input_ids"] = self._to_dev(d["input_ids"]).long()
        ctx.extras["positions"] = self._to_dev(d["positions"]).long()
        # every sequence of the step brings its whole context with it (no cached prefix, no earlier chunk)
        ctx.extras["no_prefix"] = bool(b.is_prefill and all(int(n) == int(q) for n, q in zip(b.seq_lens, q_lens)))
        if self.cache.hisparse is not None:
            tier = self.cache.hisparse
            for s, sid in zip(b.hisparse_slots, b.seq_ids):
                tier.assign(int(s), int(sid))
            ctx.hisparse = tier
            ctx.hs_slots = self._to_dev(np.asarray([s if s >= 0 else tier.scratch_slot for s in b.hisparse_slots], dtype=np.int32))
        if self.plan.needs_state_slots:
            # a sequence whose whole context arrives in this step carries no state in; unassigned slots go to the scratch slot
            slots = np.asarray([s if s >= 0 else self.cache.scratch_slot for s in b.state_slots], dtype=np.int32)
            fresh = (np.asarray(d["context_lens"]) == np.asarray(q_lens)).astype(np.int32)
            ctx.state_slots, ctx.seq_fresh = self._to_dev(slots), self._to_dev(fresh)
            ctx.conv_states, ctx.rec_states = self.cache.conv_states, self.cache.rec_states
            ctx.comp_caches, ctx.comp_kv_states, ctx.comp_score_states = self.cache.comp, self.cache.comp_kv_state, self.cache.comp_score_state
            ctx.extras["state_slots_host"] = slots.tolist()
            ctx.extras["fresh_host"] = fresh.tolist()
        return ctx

    def _dummy_context(self, is_prefill: bool) -> ForwardContext:
        """One token on the scratch page so an idle DP rank still joins every EP collective of the step."""
        dev = self.device
        sb = self.cache.scratch_block
        ctx = ForwardContext(
            is_prefill=is_prefill, num_seqs=1, num_tokens=1,
            cu_seqlens_q=torch.tensor([0, 1], dtype=torch.int32, device=dev), context_lens=torch.tensor([1], dtype=torch.int32, device=dev),
            slot_mapping=torch.tensor([sb * self.plan.block_size], dtype=torch.int64, device=dev),
            block_tables=torch.tensor([[sb]], dtype=torch.int32, device=dev), max_seqlen_q=1, max_seqlen_k=1,
            last_token_indices=torch.tensor([0], dtype=torch.int32, device=dev), q_len_uniform=1, is_dummy=True,
            kv_caches=self.cache.layers, indexer_caches=self.cache.indexer_layers, cu_seqlens_q_host=[0, 1], context_lens_host=[1])
        ctx.extras["input_ids"] = torch.zeros(1, dtype=torch.long, device=dev)
        ctx.extras["positions"] = torch.zeros(1, dtype=torch.long, device=dev)
        if self.cache.hisparse is not None:
            ctx.hisparse = self.cache.hisparse
            ctx.hs_slots = torch.tensor([self.cache.hisparse.scratch_slot], dtype=torch.int32, device=dev)
        if self.plan.needs_state_slots:
            ctx.state_slots = torch.tensor([self.cache.scratch_slot], dtype=torch.int32, device=dev)
            ctx.seq_fresh = torch.ones(1, dtype=torch.int32, device=dev)
            ctx.conv_states, ctx.rec_states = self.cache.conv_states, self.cache.rec_states
            ctx.comp_caches, ctx.comp_kv_states, ctx.comp_score_states = self.cache.comp, self.cache.comp_kv_state, self.cache.comp_score_state
            ctx.extras["state_slots_host"] = [self.cache.scratch_slot]
            ctx.extras["fresh_host"] = [1]
        return ctx

    # ---- execution -----------------------------------------------------------------------------
    # ---- vision embeddings -----------------------------------------------------------------------
    def register_vision(self, seq_id: int, prompt_token_ids, image_token_id: int, embeddings=None, pool_desc=None, slot: int = -1,
                        num_tokens: int = 0) -> int:
        """Attach the image embeddings of a request: the rows replace, in order, the embeddings of its `image_token_id`
        prompt tokens during prefill (also when the prompt is prefetched in chunks).  `embeddings` [n, hidden] directly, or
        a pool descriptor of a vision encoder (`vl.EmbeddingPool.export`) plus the slot to read.
        Parity: reference runtime/runner/vision_embed.py:33-82 (masked scatter of image rows), :84-140 (one-sided fetch)."""
        if embeddings is None:
            from ..vl.embedding_pool import EmbeddingReader
            key = id(pool_desc.get("tensor")) if isinstance(pool_desc.get("tensor"), torch.Tensor) else str(sorted(pool_desc.items(), key=str))[:256]
            readers = self.__dict__.setdefault("_vision_readers", {})
            if key not in readers:
                readers[key] = EmbeddingReader(pool_desc, self.device)
            embeddings = readers[key].fetch(slot, num_tokens, self.dtype)
        ids = np.asarray(prompt_token_ids, dtype=np.int64)
        is_img = ids == image_token_id
        if int(is_img.sum()) != embeddings.shape[0]:
            raise ValueError(f"request {seq_id}: {int(is_img.sum())} image tokens in the prompt but {embeddings.shape[0]} embedding rows")
        if embeddings.shape[1] != self.mc.hidden_size:
            raise ValueError("embedding width differs from the model's hidden size")
        self.__dict__.setdefault("_vision", {})[int(seq_id)] = (np.concatenate([[0], np.cumsum(is_img)]), is_img,
                                                                  embeddings.to(self.device, self.dtype))
        return embeddings.shape[0]

    def release_vision(self, seq_id: int) -> None:
        self.__dict__.get("_vision", {}).pop(int(seq_id), None)

    def _vision_inputs_embeds(self, b, ctx: ForwardContext):
        """inputs_embeds of a prefill step when one of its sequences carries image embeddings, else None."""
        reg = self.__dict__.get("_vision")
        if not reg or not ctx.is_prefill or not any(int(s) in reg for s in b.seq_ids):
            return None
        embed = getattr(self.model, "embed_tokens", None) or self.model.model.embed_tokens
        ids = ctx.extras["input_ids"]
        x = embed(ids).clone()
        row = 0
        for sid, q, n in zip(b.seq_ids, b.q_lens, b.seq_lens):
            ent = reg.get(int(sid))
            if ent is not None:
                prefix, is_img, emb = ent
                lo, hi = n - q, min(n, len(is_img))                     # prompt positions covered by this chunk
                if hi > lo:
                    sel = np.nonzero(is_img[lo:hi])[0]
                    if sel.size:
                        rows = torch.from_numpy(sel + row).to(x.device)
                        x.index_copy_(0, rows, emb[int(prefix[lo]): int(prefix[lo]) + sel.size])
                if n >= len(is_img):
                    reg.pop(int(sid))                                   # the whole prompt is in: the rows are no longer needed
            row += q
        return x

    @torch.inference_mode()
    def forward(self, ctx: ForwardContext) -> torch.Tensor:
        ids, pos = ctx.extras["input_ids"], ctx.extras["positions"]
        if ctx.extras.get("inputs_embeds") is not None:
            return self.model(ids, pos, ctx, inputs_embeds=ctx.extras["inputs_embeds"])
        if self.graphs is not None and not ctx.is_prefill and ctx.q_len_uniform == 1 and self.graphs.can_run(ctx):
            return self.graphs.run(ids, pos, ctx)
        if self.config.pp > 1:
            return self._forward_pp_stage(ids, pos, ctx)
        return self.model(ids, pos, ctx)

    def _forward_pp_stage(self, ids, pos, ctx: ForwardContext):
        """One stage of the prefill pipeline: receive (hidden, residual) from the previous stage, run this stage's layers,
        pass the pair on.  Only the last stage returns hidden states; the others return None."""
        from ..models.pp import pp_recv, pp_send
        d = self.dist
        inner = self.model.model
        if d.is_first_pp:
            out = inner(ids, pos, ctx)
        else:
            h, res = pp_recv(ids.numel(), self.mc.hidden_size, self.dtype, self.device, d.pp_neighbor(-1))
            out = inner(None, pos, ctx, inputs_embeds=h, residual=res)
        if d.is_last_pp:
            return out
        h, res = out
        pp_send(h, res, d.pp_neighbor(+1))
        return None

    def _check_kernel_status(self) -> None:
        """Every bounded device wait that gives up (a flag nobody raised, an mbarrier that never completed) leaves a code in
        the kernels' status words.  They are read here, right after the step's token copy already synchronised the stream,
        every `kernel_status_every` steps; a non-zero code stops the worker with an error instead of serving wrong tokens."""
        every = self.config.kernel_status_every
        if self.device.type != "cuda" or every <= 0:
            return
        self._status_steps = getattr(self, "_status_steps", 0) + 1
        if self._status_steps % every:
            return
        from ..ops import sm100
        st = sm100.kernel_status()
        if st[0] != 0:
            raise RuntimeError(f"a device wait timed out (kernel status {list(st)}): a peer GPU stopped answering or a kernel lost a hand-shake")

    # ---- file-backed KV tier (one store per worker: every rank persists its own shard of a block) ----
    def l3_open(self, root: str, capacity_blocks: int = 0) -> int:
        from .l3_store import L3Store, model_tag
        self.l3 = L3Store(self.cache, root, rank=self.dist.rank if self.dist is not None else 0, capacity_blocks=capacity_blocks,
                          tag=model_tag(self.config))
        return len(self.l3)

    def l3_exists(self, hashes: List[int]) -> List[int]:
        return self.l3.exists(hashes)

    def l3_store(self, pairs) -> int:
        return len(self.l3.store(pairs))

    def l3_load(self, pairs) -> int:
        return self.l3.load(pairs)

    def l3_stats(self) -> dict:
        return self.l3.stats()

    # ---- prefill -> decode KV push (see parallel/kv_transfer.py) -------------------------------------------------
    def pd_export_pool(self, direct: bool = False) -> dict:
        """Decode side: describe this worker's page pools, completion flags and MTP hand-off table so that a prefill worker on
        this machine can map them (`direct`: hand over the tensors themselves, for a prefill engine in the same process)."""
        from ..parallel.kv_transfer import PD_FLAGS_PER_SOURCE, PD_MAX_SOURCES, export_tensor
        if getattr(self, "pd_flags", None) is None:
            self.pd_flags = torch.zeros(PD_MAX_SOURCES * PD_FLAGS_PER_SOURCE, dtype=torch.int32, device=self.device)
        fams = []
        for f in self.cache.transfer_families():
            t = f["tensor"]
            flat = (t.view(torch.uint8) if t.dtype == torch.float8_e4m3fn else t).reshape(-1)
            fams.append({"name": f["name"], "planes": f["planes"], "plane_stride": f["plane_stride"], "page_bytes": f["page_bytes"], "by": f["by"],
                         "tensor": export_tensor(flat, direct)})
        return {"dp": self.dist.attn_dp_rank, "tp": self.dist.attn_tp_rank, "num_blocks": self.cache.num_blocks, "families": fams,
                "flags": export_tensor(self.pd_flags, direct),
                "handoff": export_tensor(self.mtp_runner.handoff, direct) if self.mtp_runner is not None else None}

    def pd_open_pool(self, key: str, pools: List[dict]) -> int:
        """Prefill side: map the pools of the decode engine `key` (those of this worker's TP rank) and check that every cache
        family has the layout of the local one.  Returns how many pools are mapped."""
        from ..parallel.kv_transfer import check_families, open_tensor
        mine = self.cache.transfer_families()
        if self.device.type == "cuda":
            torch.cuda.set_device(self.device)       # peer mappings are opened with the writing device current
        peers = getattr(self, "_pd_peers", None)
        if peers is None:
            peers = self._pd_peers = {}
        n = 0
        for p in pools:
            if p["tp"] != self.dist.attn_tp_rank:
                continue
            check_families(mine, p["families"])
            q = dict(p)
            q["families"] = [dict(f, tensor=open_tensor(f["tensor"])) for f in p["families"]]
            q["flags"] = open_tensor(p["flags"])
            q["handoff"] = open_tensor(p["handoff"]) if p.get("handoff") is not None else None
            peers[(key, p["dp"])] = q
            n += 1
        if self.device.type == "cuda":
            self._pd_counter = torch.zeros(1, dtype=torch.int32, device=self.device)
        return n

    def pd_push(self, key: str, reqs: List[dict]) -> List[int]:
        """Prefill side: queue the push of every request in `reqs` that this worker's attention-DP rank prefilled.  Per request:
        the MTP hand-off row, then one `ne_kv_push` per cache family; the last launch raises the request's flag (value
        `epoch`) in the decode GPU's memory.  Returns the bytes queued per request (0 for requests of other ranks)."""
        import ctypes as _c
        sizes = []
        for r in reqs:
            if r["src_dp"] != self.dist.attn_dp_rank:
                sizes.append(0)
                continue
            peer = self._pd_peers[(key, r["dst_dp"])]
            sb, db = r["src_blocks"], r["dst_blocks"]
            if len(sb) != len(db) or any(not (0 <= b < self.cache.num_blocks) for b in sb) or any(not (0 <= b < peer["num_blocks"]) for b in db):
                raise ValueError("kv push: page ids outside the pools")        # never hand a bad index to the kernel
            if peer["handoff"] is not None and self.mtp_runner is not None and r["src_slot"] >= 0 and r["dst_slot"] >= 0:
                peer["handoff"][r["dst_slot"]].copy_(self.mtp_runner.handoff[r["src_slot"]])
            # per-sequence state (recurrent state, compressor carries) moves by state slot, everything else by page; the
            # per-slot families come first, so the launch that raises the flag is still the last per-page one
            fams = self.cache.transfer_families()
            ss, ds = int(r.get("src_state", -1)), int(r.get("dst_state", -1))
            if any(f["by"] == "slot" for f in fams):
                n_slots = self.plan.state_slots
                if not (0 <= ss < n_slots and 0 <= ds < n_slots):
                    raise ValueError("kv push: a family with per-sequence state needs the state slots of both sides")
            total = 0
            if self.device.type != "cuda":
                for f, pf in zip(fams, peer["families"]):
                    src = (f["tensor"].view(torch.uint8) if f["tensor"].dtype == torch.float8_e4m3fn else f["tensor"]).reshape(-1).view(torch.uint8)
                    dst = pf["tensor"].view(torch.uint8) if pf["tensor"].dtype == torch.float8_e4m3fn else pf["tensor"].reshape(-1).view(torch.uint8)
                    ids = ([ss], [ds]) if f["by"] == "slot" else (sb, db)
                    for pl in range(f["planes"]):
                        for s_, d_ in zip(*ids):
                            so, do = pl * f["plane_stride"] + s_ * f["page_bytes"], pl * pf["plane_stride"] + d_ * pf["page_bytes"]
                            dst[do:do + f["page_bytes"]] = src[so:so + f["page_bytes"]]
                    total += f["planes"] * len(ids[0]) * f["page_bytes"]
                peer["flags"][r["flag"]] = r["epoch"]
                sizes.append(total)
                continue
            from ..ops import sm100 as k
            dev = self.device
            sbt = torch.tensor(sb, dtype=torch.int32).pin_memory().to(dev, non_blocking=True)
            dbt = torch.tensor(db, dtype=torch.int32).pin_memory().to(dev, non_blocking=True)
            sst = torch.tensor([max(ss, 0)], dtype=torch.int32).pin_memory().to(dev, non_blocking=True)
            dst_ = torch.tensor([max(ds, 0)], dtype=torch.int32).pin_memory().to(dev, non_blocking=True)
            fi = torch.tensor([r["flag"]], dtype=torch.int32).pin_memory().to(dev, non_blocking=True)
            for i, (f, pf) in enumerate(zip(fams, peer["families"])):
                last = i == len(fams) - 1
                src_ids, dst_ids, n_ids = (sst, dst_, 1) if f["by"] == "slot" else (sbt, dbt, len(sb))
                k._ck(k.lib().ne_kv_push(_c.c_void_p(f["tensor"].data_ptr()), _c.c_void_p(pf["tensor"].data_ptr()),
                                         _c.c_longlong(f["plane_stride"]), _c.c_longlong(pf["plane_stride"]), _c.c_int(f["page_bytes"]),
                                         k._p(src_ids), k._p(dst_ids), _c.c_int(n_ids), _c.c_int(f["planes"]), _c.c_void_p(peer["flags"].data_ptr()),
                                         k._p(fi), _c.c_int(1 if last else 0), _c.c_int(r["epoch"]), k._p(self._pd_counter), k._st()), "ne_kv_push")
                total += f["planes"] * n_ids * f["page_bytes"]
            if not sb:                       # nothing to move (a prompt that fits no page yet): the flag still has to come
                peer["flags"][r["flag"]] = r["epoch"]
            sizes.append(total)
        return sizes

    def pd_wait(self, dst_dp: int, flags: List[int], epochs: List[int], spin_limit: int = 1 << 22):
        """Decode side: bounded wait until flag `flags[i]` has reached `epochs[i]`; one bool per flag.  Workers of other
        attention-DP ranks return None.  A flag that does not come within the limit is False - the device, the stream and the
        kernels' status words are untouched."""
        if dst_dp != self.dist.attn_dp_rank:
            return None
        if getattr(self, "pd_flags", None) is None:
            return [False] * len(flags)
        if self.device.type != "cuda":
            return [int(self.pd_flags[f]) >= e for f, e in zip(flags, epochs)]
        import ctypes as _c
        from ..ops import sm100 as k
        dev = self.device
        fi = torch.tensor(flags, dtype=torch.int32).pin_memory().to(dev, non_blocking=True)
        want = torch.tensor(epochs, dtype=torch.int32).pin_memory().to(dev, non_blocking=True)
        out = torch.zeros(len(flags), dtype=torch.int32, device=dev)
        k._ck(k.lib().ne_kv_wait_each(k._p(self.pd_flags), k._p(fi), k._p(want), _c.c_int(len(flags)), k._p(out), _c.c_int(spin_limit), k._st()),
              "ne_kv_wait_each")
        return [bool(v) for v in out.tolist()]

    @torch.inference_mode()
    def run_batch(self, b) -> "C.RunnerOut":
        self.timer.start("swap")
        if b.swap_out_src:
            self.cache.swap(list(b.swap_out_src), list(b.swap_out_dst), to_host=True)
        if b.swap_in_src:
            self.cache.swap(list(b.swap_in_src), list(b.swap_in_dst), to_host=False)
        self.timer.stop()
        self.timer.start("prepare")
        with nvtx.range("step/prepare"):
            ctx = self.prepare(b)
            if not ctx.is_dummy:
                ctx.extras["inputs_embeds"] = self._vision_inputs_embeds(b, ctx)
        self.timer.stop()
        if self.mtp_runner is not None and not ctx.is_dummy:
            return self.mtp_runner.run(b, ctx)
        self.timer.forward_begin()
        with nvtx.range("step/prefill_forward" if ctx.is_prefill else "step/decode_forward"):
            hidden = self.forward(ctx)
        if hidden is None:                      # an inner pipeline stage: nothing to sample here
            self.timer.forward_end()
            return C.RunnerOut([], [])
        if ctx.is_dummy:
            if self.mtp_runner is not None:
                self.mtp_runner.run_dummy(ctx)
            self.timer.forward_end()
            return C.RunnerOut([], [])
        mask = np.asarray(b.sample_mask, dtype=bool)
        if not mask.any():
            self.timer.forward_end()
            return C.RunnerOut([], [])
        rows = ctx.last_token_indices.long()
        if not mask.all():
            rows = rows[torch.from_numpy(mask).to(rows.device)]
        with nvtx.range("step/lm_head_sample"):
            logits = self.model.compute_logits(hidden[rows])
            temps = self._to_dev(np.asarray([t for t, m in zip(b.temperatures, mask) if m], dtype=np.float32))
            tok, lp = self.sampler(logits, temps, b.any_return_logprobs)
        self.timer.forward_end()
        self.timer.start("d2h")
        with nvtx.range("step/copy_back"):
            toks = tok.tolist()
        lps = lp.tolist() if lp is not None else None
        self.d2h_bytes += tok.numel() * tok.element_size() + (lp.numel() * 4 if lp is not None else 0)
        self.timer.stop()
        self._check_kernel_status()
        if not ctx.is_prefill:
            self._last_decode = (ctx, temps)
        ids = [s for s, m in zip(b.seq_ids, mask) if m]
        return C.RunnerOut(ids, [[t] for t in toks], None if lps is None else [[x] for x in lps])

    # ---- benchmark helpers ----------------------------------------------------------------------
    @torch.inference_mode()
    def make_resident_decode_step(self):
        """A closure that repeats the most recent decode step (forward + lm_head + sampling) on inputs already on the device."""
        if self._last_decode is None:
            raise RuntimeError("run a decode step first")
        ctx, temps = self._last_decode
        ids, pos = ctx.extras["input_ids"], ctx.extras["positions"]
        rows = ctx.last_token_indices.long()

        @torch.inference_mode()
        def step():
            hidden = self.forward(ctx)
            logits = self.model.compute_logits(hidden[rows])
            return self.sampler(logits, temps, False)[0]

        return step

    @torch.inference_mode()
    def graph_step_equals_eager(self) -> bool:
        """The most recent decode step once through the captured graph and once eagerly: the sampled tokens must be the same
        (same kernels on the same inputs; a difference means the replay reads something stale)."""
        if self._last_decode is None:
            raise RuntimeError("run a decode step first")
        ctx, temps = self._last_decode
        ids, pos = ctx.extras["input_ids"], ctx.extras["positions"]
        rows = ctx.last_token_indices.long()
        a = self.sampler(self.model.compute_logits(self.forward(ctx)[rows]), torch.zeros_like(temps), False)[0]
        b = self.sampler(self.model.compute_logits(self.model(ids, pos, ctx)[rows]), torch.zeros_like(temps), False)[0]
        return bool(torch.equal(a, b))

    @torch.inference_mode()
    def count_step_launches(self) -> int:
        """Kernels of this library launched by one decode step, counted on an eager (non-graph) run of the last step."""
        from ..ops import sm100
        if self._last_decode is None:
            raise RuntimeError("run a decode step first")
        ctx, temps = self._last_decode
        before = sm100.LAUNCHES[0]
        hidden = self.model(ctx.extras["input_ids"], ctx.extras["positions"], ctx)
        logits = self.model.compute_logits(hidden[ctx.last_token_indices.long()])
        self.sampler(logits, temps, False)
        torch.cuda.synchronize()
        return sm100.LAUNCHES[0] - before

    def run_from_bytes(self, blob: bytes) -> bytes:
        return self.run_batch(C.RunnerIn.from_bytes(blob)).to_bytes()

    # ---- profiler control ----------------------------------------------------------------------
    def start_profiler(self, trace_name: str = "trace") -> bool:
        if self._profiler is not None or not self.config.profiler_dir:
            return False
        acts = [torch.profiler.ProfilerActivity.CPU]
        if self.device.type == "cuda":
            acts.append(torch.profiler.ProfilerActivity.CUDA)
        self._profiler = (torch.profiler.profile(activities=acts), trace_name)
        self._profiler[0].start()
        return True

    def stop_profiler(self) -> Optional[str]:
        if self._profiler is None:
            return None
        prof, name = self._profiler
        prof.stop()
        os.makedirs(self.config.profiler_dir, exist_ok=True)
        path = os.path.join(self.config.profiler_dir, f"{name}.rank{self.rank}.json")
        prof.export_chrome_trace(path)
        self._profiler = None
        return path

    def get_step_timing(self) -> Dict[str, float]:
        out = dict(self.timer.phases)
        out["forward_ms_last"] = self.timer.last_forward_ms
        return out
