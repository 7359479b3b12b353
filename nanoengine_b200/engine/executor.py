"""Executors: launch one worker per GPU and fan calls out to them.

* ``InprocExecutor``  - the single worker lives in the controller process (world size 1).
* ``MultiprocExecutor`` - one spawned process per rank; each joins ``torch.distributed`` (NCCL for device
  collectives + gloo for host control, or gloo only on CPU) and serves calls over a pipe.  A watchdog
  notices a dead worker and fails the pending call instead of hanging the controller.

Parity: reference executor/ray_executor.py:100-482 (collective_rpc :311, run_batch_bytes_async :407,
KV-block count = min over workers :443); the Ray / RDMA-RPC transports are replaced by pipes on one box.
"""
from __future__ import annotations

import os
import socket
import traceback
from typing import Any, List, Optional, Sequence

import torch

from ..config import Config


class ExecutorError(RuntimeError):
    pass


_LEFT_KEY = "nanoengine/ranks_left"


class InprocExecutor:
    in_process = True          # the workers' tensors are reachable from the controller's address space

    def __init__(self, config: Config):
        from ..runtime.model_runner import ModelRunner
        self.config = config
        self.world_size = 1
        self.runner = ModelRunner(config, 0, 1)

    def collective_rpc(self, method: str, *args, **kw) -> List[Any]:
        return [getattr(self.runner, method)(*args, **kw)]

    def rank_rpc(self, method: str, per_rank_arg: Sequence[Any]) -> List[Any]:
        return [getattr(self.runner, method)(per_rank_arg[0])]

    def run_batches(self, blobs: Sequence[bytes]) -> List[bytes]:
        return [self.runner.run_from_bytes(blobs[0])]

    def run_batches_pipelined(self, waves):
        return [self.run_batches(w) for w in waves]

    def shutdown(self):
        self.runner = None


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker_main(rank: int, world_size: int, config_dict: dict, port: int, conn, use_cuda: bool):
    try:
        import torch.distributed as dist
        from ..config import Config as _Config
        from ..runtime.model_runner import ModelRunner
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        os.environ["RANK"], os.environ["WORLD_SIZE"], os.environ["LOCAL_RANK"] = str(rank), str(world_size), str(rank)
        cfg = _Config.from_dict(config_dict)
        if use_cuda:
            torch.cuda.set_device(rank)
            dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=world_size, device_id=torch.device(f"cuda:{rank}"))
        else:
            torch.set_num_threads(max(1, (os.cpu_count() or 2) // world_size))
            dist.init_process_group("gloo", rank=rank, world_size=world_size)
        runner = ModelRunner(cfg, rank, world_size, device=f"cuda:{rank}" if use_cuda else "cpu")
        conn.send(("ready", None))
        while True:
            msg = conn.recv()
            if msg is None:
                break
            method, args, kw = msg
            try:
                conn.send(("ok", getattr(runner, method)(*args, **kw)))
            except Exception as e:  # report and keep serving: the controller decides what to do
                conn.send(("err", f"{type(e).__name__}: {e}\n{traceback.format_exc()}"))
        dist.destroy_process_group()
    except Exception as e:
        try:
            conn.send(("err", f"worker {rank} failed to start: {e}\n{traceback.format_exc()}"))
        except Exception:
            pass


class MultiprocExecutor:
    in_process = False

    def __init__(self, config: Config, timeout_s: float = 600.0):
        import torch.multiprocessing as mp
        self.config = config
        self.world_size = config.world_size
        self.timeout_s = timeout_s
        use_cuda = config.device == "cuda" or (config.device == "auto" and torch.cuda.is_available())
        if use_cuda and torch.cuda.device_count() < self.world_size:
            raise ExecutorError(f"layout needs {self.world_size} GPUs, {torch.cuda.device_count()} visible")
        ctx = mp.get_context("spawn")
        port = _free_port()
        self.procs, self.conns = [], []
        cd = config.to_dict()
        for r in range(self.world_size):
            parent, child = ctx.Pipe()
            p = ctx.Process(target=_worker_main, args=(r, self.world_size, cd, port, child, use_cuda), daemon=True)
            p.start()
            self.procs.append(p)
            self.conns.append(parent)
        for r in range(self.world_size):
            self._recv(r)

    def _recv(self, r: int):
        conn, p = self.conns[r], self.procs[r]
        waited = 0.0
        while not conn.poll(0.5):
            waited += 0.5
            if not p.is_alive():
                raise ExecutorError(f"worker {r} died (exit code {p.exitcode})")
            if waited > self.timeout_s:
                raise ExecutorError(f"worker {r} did not answer within {self.timeout_s}s")
        try:
            status, val = conn.recv()
        except EOFError:
            raise ExecutorError(f"worker {r} closed its pipe")
        if status == "err":
            raise ExecutorError(val)
        return val

    def _send(self, r: int, msg) -> None:
        try:
            self.conns[r].send(msg)
        except (BrokenPipeError, OSError) as e:
            raise ExecutorError(f"worker {r} is gone (exit code {self.procs[r].exitcode}): {e}")

    def collective_rpc(self, method: str, *args, **kw) -> List[Any]:
        for r in range(self.world_size):
            self._send(r, (method, args, kw))
        return [self._recv(r) for r in range(self.world_size)]

    def rank_rpc(self, method: str, per_rank_arg: Sequence[Any]) -> List[Any]:
        """Like collective_rpc, with a different single argument for every worker."""
        for r in range(self.world_size):
            self._send(r, (method, (per_rank_arg[r],), {}))
        return [self._recv(r) for r in range(self.world_size)]

    def _batch_index(self, rank: int) -> int:
        s = self.config.parallel_spec()
        return (rank // (s.attention_sp * s.attention_tp)) % s.attention_dp

    def run_batches(self, blobs: Sequence[bytes]) -> List[bytes]:
        """blobs: one per attention-DP rank.  Returns one result per DP rank (from attention-TP rank 0)."""
        s = self.config.parallel_spec()
        for r in range(self.world_size):
            self._send(r, ("run_from_bytes", (blobs[self._batch_index(r)],), {}))
        outs = [self._recv(r) for r in range(self.world_size)]
        tp = s.attention_sp * s.attention_tp
        per_stage = self.world_size // s.pp
        last_stage = (s.pp - 1) * per_stage
        return [outs[last_stage + d * tp] for d in range(s.attention_dp)]

    def run_batches_pipelined(self, waves: Sequence[Sequence[bytes]]) -> List[List[bytes]]:
        """Submit every wave of micro-batches before collecting any result, so pipeline stages overlap."""
        s = self.config.parallel_spec()
        for wave in waves:
            for r in range(self.world_size):
                self._send(r, ("run_from_bytes", (wave[self._batch_index(r)],), {}))
        tp = s.attention_sp * s.attention_tp
        last_stage = (s.pp - 1) * (self.world_size // s.pp)
        out = []
        for _ in waves:
            outs = [self._recv(r) for r in range(self.world_size)]
            out.append([outs[last_stage + d * tp] for d in range(s.attention_dp)])
        return out

    def alive(self) -> List[bool]:
        return [p.is_alive() for p in self.procs]

    def shutdown(self):
        for c, p in zip(self.conns, self.procs):
            try:
                if p.is_alive():
                    c.send(None)
            except Exception:
                pass
        for p in self.procs:
            p.join(timeout=10)
            if p.is_alive():
                p.terminate()
        self.procs, self.conns = [], []


class SpmdExecutor:
    """One engine per rank, launched by torchrun (one process per GPU).  Every rank schedules the requests of its own
    attention-DP shard; ranks only meet inside the model's collectives, so before each step they agree (one tiny host
    all-reduce) whether anybody has work - a rank without work then runs a dummy batch to keep the collectives matched."""

    in_process = True

    def __init__(self, config: Config):
        import torch.distributed as dist
        from ..runtime.model_runner import ModelRunner
        self.config = config
        self.rank = int(os.environ.get("RANK", "0"))
        self.world_size = int(os.environ.get("WORLD_SIZE", "1"))
        if self.world_size != config.world_size:
            raise ExecutorError(f"layout needs {config.world_size} ranks, launched with {self.world_size}")
        use_cuda = config.device == "cuda" or (config.device == "auto" and torch.cuda.is_available())
        local = int(os.environ.get("LOCAL_RANK", self.rank))
        if self.world_size > 1 and not dist.is_initialized():
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            if use_cuda:
                torch.cuda.set_device(local)
                dist.init_process_group("cpu:gloo,cuda:nccl", rank=self.rank, world_size=self.world_size, device_id=torch.device(f"cuda:{local}"))
            else:
                dist.init_process_group("gloo", rank=self.rank, world_size=self.world_size)
        self.runner = ModelRunner(config, self.rank, self.world_size, device=f"cuda:{local}" if use_cuda else "cpu")
        self._host_group = None
        self._store = None
        if self.world_size > 1:
            import datetime
            self._host_group = dist.new_group(list(range(self.world_size)), backend="gloo",
                                              timeout=datetime.timedelta(seconds=config.peer_timeout_s))
            try:
                self._store = dist.distributed_c10d._get_default_store()
            except Exception:
                self._store = None

    def collective_rpc(self, method: str, *args, **kw) -> List[Any]:
        return [getattr(self.runner, method)(*args, **kw)]

    def agree(self, has_work: bool, is_prefill: bool):
        """(anybody has work, anybody prefills) across all ranks."""
        if self.world_size == 1:
            return has_work, is_prefill
        import torch.distributed as dist
        # Failure detection happens here, on the host and before anything is launched: a rank that left announced it in the
        # job's store; one that died silently makes the rendezvous fail or run into the group's timeout.  Either way this
        # rank stops stepping with an error instead of entering device collectives its peer will never join.
        try:
            if self._store is not None and int(self._store.add(_LEFT_KEY, 0)) > 0:
                raise ExecutorError("a peer rank has left the job")
            t = torch.tensor([int(has_work), int(is_prefill)], dtype=torch.int32)
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self._host_group)
        except ExecutorError:
            raise
        except Exception as e:
            raise ExecutorError(f"a peer rank stopped answering the per-step rendezvous: {e}") from e
        return bool(t[0]), bool(t[1])

    def min_over_ranks(self, v: int) -> int:
        if self.world_size == 1:
            return v
        import torch.distributed as dist
        t = torch.tensor([v], dtype=torch.int64)
        dist.all_reduce(t, op=dist.ReduceOp.MIN, group=self._host_group)
        return int(t[0])

    def run_batches(self, blobs: Sequence[bytes]) -> List[bytes]:
        return [self.runner.run_from_bytes(blobs[0])]

    def shutdown(self):
        """Leaves between steps (nothing of this rank is in flight) and says so, so the peers stop at their next rendezvous."""
        if self.runner is not None and self._store is not None:
            try:
                if torch.cuda.is_available() and self.runner.device.type == "cuda":
                    torch.cuda.synchronize(self.runner.device)
                self._store.add(_LEFT_KEY, 1)
            except Exception:
                pass
        self.runner = None


def build_executor(config: Config):
    backend = config.executor_backend
    if backend == "spmd":
        return SpmdExecutor(config)
    if backend == "auto":
        backend = "inproc" if config.world_size == 1 else "mp"
    if backend == "inproc":
        if config.world_size != 1:
            raise ValueError("the in-process executor runs exactly one worker")
        return InprocExecutor(config)
    if backend == "mp":
        return MultiprocExecutor(config)
    raise ValueError(f"unknown executor_backend {backend}")
