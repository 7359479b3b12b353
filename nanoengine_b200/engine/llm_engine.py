"""The engine controller: native scheduler + executor + the step loop.

Parity: reference engine/llm_engine.py - _build_executor :16-25, __init__ :29-59, step :386-406,
_run_scheduled_step :175-222, profiler fan-out :95-122, update_weights :124-148; engine/scheduler.py:19-143
(SchedulerConfig from Config and the model's cache plan, token budget).
"""
from __future__ import annotations

import time
from typing import Dict, Iterable, List, Optional

from .._native import _core as C
from ..config import Config
from ..utils.logging import get_logger
from .executor import build_executor

logger = get_logger("nanoengine.engine")

_ROUTING = {"round_robin": C.ROUND_ROBIN, "least_batch": C.LEAST_BATCH, "least_cache": C.LEAST_CACHE, "affinity": C.AFFINITY}
_MODE = {"hybrid": C.MODE_HYBRID, "prefill": C.MODE_PREFILL, "decode": C.MODE_DECODE}


def scheduler_token_budget(config: Config) -> int:
    """Per-step prefill token budget; a prefill pipeline keeps `pp` micro-batches in flight."""
    return config.max_num_batched_tokens * max(1, config.pp)


def build_scheduler_config(config: Config, num_blocks: int, plan_bits: int) -> "C.SchedulerConfig":
    sc = C.SchedulerConfig()
    sc.num_blocks = num_blocks
    sc.num_host_blocks = config.num_host_kvcache_blocks
    sc.block_size = config.kvcache_block_size
    sc.max_num_seqs = config.max_num_seqs
    sc.max_num_batched_tokens = scheduler_token_budget(config)
    sc.max_model_len = config.max_model_len
    sc.attention_dp = 1 if config.executor_backend == "spmd" else config.attention_dp
    sc.mode = _MODE[config.mode]
    sc.num_speculative_tokens = config.num_speculative_tokens
    sc.enable_prefix_caching = config.enable_prefix_caching
    sc.enable_chunked_prefill = config.enable_chunked_prefill
    sc.routing = _ROUTING[config.routing_strategy]
    sc.cache_plan = plan_bits
    sc.num_handoff_slots = config.max_num_seqs if config.num_speculative_tokens > 0 else 0
    sc.num_hisparse_slots = config.max_num_seqs if config.enable_hisparse else 0
    sc.num_state_slots = config.max_num_seqs if (plan_bits & (C.PLAN_GDN | C.PLAN_CSA)) else 0   # one state slot per running sequence
    sc.eos_token_ids = config.model_config.eos_ids()
    sc.engine_id = config.engine_id
    return sc


def _dummy_batch(is_prefill: bool):
    """The batch an idle rank runs so that it joins every collective of the step: no sequences (the wire form wants the
    offsets table of an empty batch, one zero), flagged so the worker substitutes one token on the scratch page."""
    b = C.RunnerIn()
    b.is_dummy, b.is_prefill = True, is_prefill
    b.block_offsets = [0]
    return b


class _NoCopyMigrator:
    """Migrator of a dummy-prefill decode engine: every import "succeeds" without moving a byte."""

    def pull(self, blobs):
        ids = []
        for blob in blobs:
            ids += list(C.MigrationIn.from_bytes(blob).seq_ids)
        return ids, [], 0


class LLMEngine:
    def __init__(self, config: Config, executor=None):
        self.config = config
        self.executor = executor or build_executor(config)
        self.executor.collective_rpc("init_model")
        counts = self.executor.collective_rpc("profile_num_blocks")
        self.num_blocks = int(min(counts))
        self.spmd = config.executor_backend == "spmd"
        if self.spmd:
            self.num_blocks = self.executor.min_over_ranks(self.num_blocks)
        if self.num_blocks < 1:
            raise RuntimeError("no memory left for the KV cache; lower gpu_memory_utilization or the model size")
        from ..runtime.cache import make_cache_plan
        plan = make_cache_plan(config.model_config, config.resolved_kv_dtype(), config.kvcache_block_size, config.attention_tp,
                               use_indexer=config.use_nsa(), hisparse_rows=config.hisparse_device_buffer_size if config.enable_hisparse else 0)
        self.scheduler = C.Scheduler(build_scheduler_config(config, self.num_blocks, plan.plan_bits()))
        self.executor.collective_rpc("allocate_kvcache", self.num_blocks)
        self._next_seq_id = 1
        self.migrator = None   # set by the PD layer (disagg.KVMigrator)
        self.endpoint = None   # ZMQ endpoint of the engine process serving this engine, once it has one (published with the description)
        self._pd_connect = None        # connector of a prefill engine found through the control plane (tests substitute it)
        self._pd_unresolved = set()
        # file-backed third KV tier: needs the prefix cache (blocks are found by their chained hash) and one block pool
        self.l3_enabled = False
        if config.l3_dir and config.enable_prefix_caching:
            if config.attention_dp > 1 and not self.spmd:
                logger.warning("l3_dir is ignored: the file-backed KV tier needs one scheduler per attention-DP rank (executor_backend=spmd)")
            else:
                self.executor.collective_rpc("l3_open", config.l3_dir, config.l3_capacity_blocks)
                self.scheduler.set_commit_log(True)
                self.l3_enabled = True

    # ---- requests ----------------------------------------------------------------------------
    def add_request_payload(self, payload: bytes) -> int:
        return self.scheduler.add_request_bytes(payload)

    def add_request(self, prompt_token_ids: List[int], sampling_params=None, seq_id: Optional[int] = None, affinity_key: int = 0) -> int:
        if seq_id is None:
            seq_id = self._next_seq_id
        self._next_seq_id = max(self._next_seq_id, seq_id) + 1
        sp = sampling_params or C.SamplingParams()
        if self.config.dummy_prefill:
            # a decode engine without a prefill peer: the prompt arrives as if it had been migrated, its cache rows stay what
            # the (zero-initialised) cold tier holds and its first token is made up; the serving flow, slot handling and graph
            # replay are exercised, the text is meaningless (reference docs/hisparse-design.md, "Dummy-prefill flow")
            m = C.RequestMigrate()
            m.seq_id, m.token_ids, m.prompt_len = seq_id, list(prompt_token_ids) + [int(prompt_token_ids[-1])], len(prompt_token_ids)
            m.num_computed, m.sampling_params, m.affinity_key = len(prompt_token_ids), sp, affinity_key
            m.migrate_block_table, m.migrate_engine_id, m.block_size = [], "dummy-prefill", self.config.kvcache_block_size
            if self.migrator is None:
                self.migrator = _NoCopyMigrator()
            return self.scheduler.add_request_bytes(m.to_bytes())
        if self.l3_enabled:
            self._l3_import(prompt_token_ids)
        return self.scheduler.add_request(C.RequestIn(seq_id, list(prompt_token_ids), sp, affinity_key))

    def add_vision_request(self, prompt_token_ids: List[int], image_token_id: int, embeddings=None, vision_slot=None, pool_desc=None,
                           sampling_params=None, seq_id: Optional[int] = None) -> int:
        """A request whose `image_token_id` prompt tokens stand for image embeddings: given directly ([n, hidden]) or as a slot of
        a vision encoder's pool (`vl.EncoderEngine.encode` + `engine_info()["pool"]`).  The workers splice the rows in during
        prefill.  Parity: reference engine/llm_component.py:285-340 + runtime/runner/model_runner.py:1557-1573, :1886-1890."""
        if seq_id is None:
            seq_id = self._next_seq_id
        slot, ntok = (int(vision_slot.slot), int(vision_slot.num_tokens)) if vision_slot is not None else (-1, 0)
        self.executor.collective_rpc("register_vision", seq_id, list(prompt_token_ids), int(image_token_id), embeddings, pool_desc, slot, ntok)
        self._next_seq_id = max(self._next_seq_id, seq_id) + 1
        sp = sampling_params or C.SamplingParams()
        return self.scheduler.add_request(C.RequestIn(seq_id, list(prompt_token_ids), sp, 0, [slot] if slot >= 0 else None))

    # ---- file-backed KV tier ------------------------------------------------------------------
    def _l3_import(self, prompt_token_ids: List[int]) -> int:
        """Bring the prompt's leading blocks that only the file tier still holds back into the device prefix cache."""
        from ..runtime.l3_store import prompt_block_hashes
        hashes = prompt_block_hashes(prompt_token_ids, self.config.kvcache_block_size)
        if not hashes:
            return 0
        stored = None
        for got in self.executor.collective_rpc("l3_exists", hashes):       # a block counts only if every worker has its shard
            stored = set(got) if stored is None else stored & set(got)
        run = []
        for h in hashes:
            if not (self.scheduler.has_cached_hash(0, h) or h in stored):
                break
            run.append(h)
        if not any(h in stored and not self.scheduler.has_cached_hash(0, h) for h in run):
            return 0
        ids = self.scheduler.begin_import(0, run)
        run = run[:len(ids)]
        pairs = [(h, b) for h, b in zip(run, ids) if b >= 0]
        ok = True
        try:
            self.executor.collective_rpc("l3_load", pairs)
        except Exception as e:                                              # a vanished file: the blocks stay unpublished
            logger.warning("L3 import failed, recomputing instead: %s", e)
            ok = False
        self.scheduler.finish_import(0, run, ids, ok)
        return len(pairs) if ok else 0

    def _l3_persist(self) -> None:
        pairs = self.scheduler.take_committed(0)
        if pairs:
            self.executor.collective_rpc("l3_store", pairs)

    def abort(self, seq_id: int) -> bool:
        return self.scheduler.abort(seq_id)

    def is_finished(self) -> bool:
        return self.scheduler.is_finished()

    # ---- the step ------------------------------------------------------------------------------
    def step(self) -> List["C.StepOut"]:
        res = self.scheduler.schedule()
        if res.migrations:
            self._run_migrations(res)
        if self.spmd:
            any_work, any_prefill = self.executor.agree(res.has_work, res.has_work and res.is_prefill)
            if any_work and not res.has_work:
                self.executor.run_batches([_dummy_batch(any_prefill).to_bytes()])
                return []
        if not res.has_work:
            return []
        t0 = time.perf_counter()
        if self.config.pp > 1 and res.is_prefill:
            outs = self._run_static_pp_prefill_pipeline(res)
        else:
            outs = self.executor.run_batches(self.scheduler.serialize_run_batches())
        ms = (time.perf_counter() - t0) * 1e3
        step_outs = self.scheduler.postprocess_runner_out_bytes(outs, ms)
        if self.l3_enabled:
            self._l3_persist()
        every = self.config.status_log_interval_s
        if every > 0 and t0 - getattr(self, "_status_logged_at", 0.0) >= every:
            self._status_logged_at = t0
            logger.info(self.scheduler.status_line(self.config.mode))
        return step_outs

    def _run_static_pp_prefill_pipeline(self, res) -> List[bytes]:
        """Split each DP rank's prefill batch into `pp` micro-batches and keep them all in flight: every worker receives
        the micro-batches in order, so stage s works on micro-batch m while stage s+1 works on m-1."""
        from ..models.pp import split_batch
        depth = self.config.pp
        per_dp = [split_batch(C.RunnerIn.from_bytes(b), depth) for b in self.scheduler.serialize_run_batches()]
        rounds = max(len(m) for m in per_dp)
        waves = []
        for r in range(rounds):
            wave = []
            for mbs in per_dp:
                if r < len(mbs):
                    wave.append(mbs[r].to_bytes())
                else:
                    wave.append(_dummy_batch(True).to_bytes())
            waves.append(wave)
        results = self.executor.run_batches_pipelined(waves)
        merged = []
        for d in range(len(per_dp)):
            ids, toks, lps = [], [], []
            for r in range(rounds):
                o = C.RunnerOut.from_bytes(results[r][d])
                ids.extend(o.seq_ids); toks.extend(o.token_ids)
            merged.append(C.RunnerOut(ids, toks).to_bytes())
        return merged

    def _resolve_pd_peers(self, blobs) -> None:
        """Decode engines: a sequence arrives from a prefill engine this engine has no connection to yet.  With a control plane
        configured, look the engine's description up there (it names the ZMQ endpoint of its engine process) and connect: the
        decode workers publish their pools to it, as they do at start-up for the peers `pd_peers` lists.
        Parity: reference engine/llm_component.py `_fetch_peer_info_from_ctrl` / `set_peer_info`."""
        if not self.config.ctrl_address:
            return
        eids = {str(e) for b in blobs for e in (getattr(C.MigrationIn.from_bytes(b), "remote_engine_ids", None) or [])}
        for eid in sorted(eids):
            known = self.migrator is not None and eid in getattr(self.migrator, "peers", {})
            if known or not eid or eid in self._pd_unresolved:
                continue
            from ..server.ctrl import fetch_engine
            info = fetch_engine(self.config.ctrl_address, eid)
            if not info or not info.get("endpoint"):
                self._pd_unresolved.add(eid)          # asked once: a request from it fails by itself, the engine keeps serving
                logger.warning("prefill engine %s is not known to the control plane %s", eid, self.config.ctrl_address)
                continue
            connect = self._pd_connect
            if connect is None:
                from ..parallel.kv_transfer import connect_remote as connect
            connect(self, eid, info["endpoint"])
            logger.info("connected to prefill engine %s at %s", eid, info["endpoint"])

    def _run_migrations(self, res) -> None:
        blobs = self.scheduler.serialize_migrate_batches()
        self._resolve_pd_peers(blobs)
        if self.migrator is None:
            raise RuntimeError("received a migrated request but no KV migrator is attached to this engine")
        t0 = time.perf_counter()
        ok_ids, bad_ids, nbytes = self.migrator.pull(blobs)
        self.scheduler.record_transfer((time.perf_counter() - t0) * 1e3, nbytes)
        if ok_ids:
            self.scheduler.complete_migration(ok_ids, True)
        if bad_ids:
            self.scheduler.complete_migration(bad_ids, False)

    # ---- PD ------------------------------------------------------------------------------------
    def export_to_be_migrated(self):
        return self.scheduler.export_to_be_migrated()

    def free_to_be_migrated_ids(self, ids: Iterable[int]) -> int:
        return self.scheduler.free_to_be_migrated(list(ids))

    # ---- control -------------------------------------------------------------------------------
    def start_profiler(self, trace_name: str = "trace") -> bool:
        if not trace_name or any(c in trace_name for c in "/\\") or ".." in trace_name:
            raise ValueError("trace name must be a plain file stem")
        return all(self.executor.collective_rpc("start_profiler", trace_name))

    def stop_profiler(self) -> List[Optional[str]]:
        return self.executor.collective_rpc("stop_profiler")

    def update_weights(self, named_tensors_or_path) -> int:
        """Swap weights in place (live update).  Accepts a checkpoint directory or an iterable of (name, tensor)."""
        n = min(self.executor.collective_rpc("update_weights", named_tensors_or_path))
        self.scheduler.reset_prefix_cache()      # cached KV was computed with the old weights
        return n

    def export_weights(self, direct: bool = False) -> List[Dict]:
        """Per-worker descriptors of the weights this engine serves (see ModelRunner.export_weights)."""
        return self.executor.collective_rpc("export_weights", direct)

    def pull_weights(self, per_worker: List[Dict]) -> int:
        """Live update from a peer engine with the same layout: worker i copies the tensors of the peer's worker i."""
        if len(per_worker) != self.executor.world_size:
            raise ValueError("the peer engine has a different number of workers")
        if self.executor.world_size == 1:
            n = self.executor.collective_rpc("pull_weights", per_worker[0])[0]
        else:
            n = min(self.executor.rank_rpc("pull_weights", per_worker))
        self.scheduler.reset_prefix_cache()
        return n

    def metrics_prometheus(self) -> str:
        return self.scheduler.metrics_prometheus()

    def metrics_summary(self) -> Dict:
        return self.scheduler.metrics_summary()

    def engine_info(self) -> Dict:
        c = self.config
        return {"id": c.engine_id, "role": c.mode, "world_size": c.world_size, "num_blocks": self.num_blocks,
                "host": c.host, "port": c.port, "max_num_seqs": c.max_num_seqs, "attention_dp": c.attention_dp,
                "attention_sp": c.attention_sp, "attention_tp": c.attention_tp, "pp": c.pp,
                "num_hidden_layers": c.model_config.num_hidden_layers, "block_size": c.kvcache_block_size,
                "architecture": c.model_config.architecture, "kv_cache_dtype": c.resolved_kv_dtype(),
                "mtp_num_kv_layers": max(1, c.model_config.num_nextn_predict_layers) if c.num_speculative_tokens else 0,
                "endpoint": getattr(self, "endpoint", None) or c.engine_endpoint}

    def shutdown(self):
        self.executor.shutdown()
