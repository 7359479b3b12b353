"""Third KV tier: one file per KV block on a shared or local file system, keyed by the block's chained token hash.

A block file holds the block's bytes of every cache family of every layer (``KVCache.block_views``), preceded by a 32-byte
header that names the layout AND the weights the KV was computed with (a model tag plus a generation counter that every
live weight update bumps), so a file written under another cache plan, another checkpoint of the same shape or an older
weight version is rejected instead of being served as a prefix hit.
Files are written to a temporary name and renamed, so a reader never sees a partial block.  The native ``L3Index`` keeps
the set of stored hashes in LRU order; with a capacity it reports the hash to drop and the store deletes its file.

The engine side (``LLMEngine``) persists freshly published prefix-cache blocks after every step and, before a request is
queued, imports the blocks of its prompt that the device prefix cache no longer holds.

Parity: reference runtime/disagg/storage/l3_hf3fs.py:37-259 (per-block files named by the 16-hex-digit hash under a
per-rank directory, `exists` / `store` / `load` / `stats`, missing file on load is an error) and rust/src/l3.rs:1-497
(block index).  The reference moves bytes with the 3FS USRBIO ring; this store uses positional POSIX reads and writes
through a pinned staging buffer, which works on any mount.
"""
from __future__ import annotations

import hashlib
import os
import struct
import time
from typing import Iterable, List, Sequence, Tuple

import torch

from .._native import _core as C

_MAGIC = b"NEL3BLK1"


def model_tag(config) -> str:
    """Identity of the weights an engine serves, for the block-file header: the checkpoint directory with the names, sizes and
    modification times of its weight files, or (random-init runs) the model shape and the seed."""
    import json
    if getattr(config, "dummy_weight", False) or not os.path.isdir(str(config.model)):
        return "dummy:" + json.dumps(config.model_config.to_dict(), sort_keys=True, default=str) + f":seed{config.seed}"
    root = os.path.abspath(config.model)
    files = []
    for name in sorted(os.listdir(root)):
        if name.endswith((".safetensors", ".json")):
            st = os.stat(os.path.join(root, name))
            files.append((name, st.st_size, st.st_mtime_ns))
    return f"ckpt:{root}:{files!r}"


class L3Store:
    def __init__(self, cache, root: str, rank: int = 0, capacity_blocks: int = 0, tag: str = ""):
        self.cache = cache
        self.dir = os.path.join(root, f"rank{rank}")
        os.makedirs(self.dir, exist_ok=True)
        self.views = cache.block_views
        probe = self.views(0)
        self.segments = [int(v.numel() * v.element_size()) for v in probe]
        self.block_nbytes = sum(self.segments)
        self._desc = repr([(tuple(v.shape), str(v.dtype)) for v in probe]).encode()
        self._tag = tag.encode()
        self.generation = self._read_generation()
        if self.generation > 0:
            # blocks left by a previous process after a live weight update: those weights existed only in that process' memory,
            # this one loaded the checkpoint again, so they match nothing that can be served now
            self._purge_files()
            self._write_generation(0)
        self._set_header()
        pin = cache.device.type == "cuda"
        self.staging = torch.empty(self.block_nbytes, dtype=torch.uint8, pin_memory=pin)
        self._capacity = capacity_blocks
        self.index = C.L3Index(capacity_blocks)
        self.bytes_stored = self.bytes_loaded = 0
        self.n_store = self.n_load = self.n_evicted = 0
        self.t_store = self.t_load = 0.0
        self._recover()

    # ---- identity of the stored KV ----
    def _gen_path(self) -> str:
        return os.path.join(self.dir, "GENERATION")

    def _read_generation(self) -> int:
        try:
            with open(self._gen_path()) as f:
                return int(f.read().strip() or 0)
        except (OSError, ValueError):
            return 0

    def _set_header(self):
        self.fingerprint = hashlib.sha256(self._desc + b"|" + self._tag + b"|" + str(self.generation).encode()).digest()[:16]
        self.header = _MAGIC + struct.pack("<Q", self.block_nbytes) + self.fingerprint

    def bump_generation(self) -> int:
        """The weights changed in place: every stored block is stale.  Moves to the next generation (persisted: a later process
        that finds a non-zero generation knows the directory holds blocks of weights it cannot have), forgets the index and
        deletes the block files."""
        self._write_generation(self.generation + 1)
        self._set_header()
        self.index = C.L3Index(self._capacity)
        self._purge_files()
        return self.generation

    def _write_generation(self, g: int):
        self.generation = g
        tmp = self._gen_path() + f".tmp{os.getpid()}"
        with open(tmp, "w") as f:
            f.write(str(g))
        os.replace(tmp, self._gen_path())

    def _purge_files(self):
        for name in os.listdir(self.dir):
            if name.endswith(".kv"):
                try:
                    os.unlink(os.path.join(self.dir, name))
                except OSError:
                    pass

    # ---- layout ----
    def _path(self, h: int) -> str:
        return os.path.join(self.dir, f"{h & 0xFFFFFFFFFFFFFFFF:016x}.kv")

    def _recover(self):
        """Rebuild the index from the directory (oldest first, so LRU order survives a restart); drop foreign files."""
        want = len(self.header) + self.block_nbytes
        entries = []
        for name in os.listdir(self.dir):
            if not name.endswith(".kv"):
                continue
            p = os.path.join(self.dir, name)
            try:
                st = os.stat(p)
                if st.st_size != want:
                    continue
                with open(p, "rb") as f:
                    if f.read(len(self.header)) != self.header:
                        continue
                entries.append((st.st_mtime, int(name[:-3], 16)))
            except (OSError, ValueError):
                continue
        for _, h in sorted(entries):
            self._index_insert(h)

    def _index_insert(self, h: int):
        ev = self.index.insert(h, 0)
        if ev:
            self.n_evicted += 1
            try:
                os.unlink(self._path(ev))
            except OSError:
                pass

    # ---- public API ----
    def __len__(self) -> int:
        return len(self.index)

    def exists(self, hashes: Iterable[int]) -> List[int]:
        return [h for h in hashes if self.index.contains(h)]

    def match(self, hashes: Sequence[int]) -> int:
        """Length of the leading run of `hashes` that is stored."""
        return self.index.match(list(hashes))

    def store(self, pairs: Sequence[Tuple[int, int]], skip_existing: bool = True) -> List[int]:
        """Persist (hash, device block id) pairs; returns the hashes now durable."""
        done = []
        for h, bid in pairs:
            if skip_existing and self.index.contains(h):
                done.append(h)
                continue
            t0 = time.monotonic()
            off = 0
            for v, n in zip(self.views(bid), self.segments):
                self.staging[off:off + n].copy_(v.contiguous().view(torch.uint8).reshape(-1), non_blocking=True)
                off += n
            if self.cache.device.type == "cuda":
                torch.cuda.current_stream().synchronize()
            tmp = self._path(h) + f".tmp{os.getpid()}"
            fd = os.open(tmp, os.O_CREAT | os.O_WRONLY | os.O_TRUNC, 0o644)
            try:
                os.pwrite(fd, self.header, 0)
                buf = memoryview(self.staging.numpy())
                pos = 0
                while pos < self.block_nbytes:
                    pos += os.pwrite(fd, buf[pos:], len(self.header) + pos)
            finally:
                os.close(fd)
            os.replace(tmp, self._path(h))
            self._index_insert(h)
            self.bytes_stored += self.block_nbytes
            self.n_store += 1
            self.t_store += time.monotonic() - t0
            done.append(h)
        return done

    def load(self, pairs: Sequence[Tuple[int, int]]) -> int:
        """Fill device blocks from their files.  A missing or foreign file raises: the caller must not publish the block."""
        n_ok = 0
        for h, bid in pairs:
            p = self._path(h)
            t0 = time.monotonic()
            try:
                fd = os.open(p, os.O_RDONLY)
            except FileNotFoundError:
                self.index.erase(h)
                raise FileNotFoundError(f"L3 block {h:#018x} is not at {p}")
            try:
                if os.pread(fd, len(self.header), 0) != self.header:
                    raise ValueError(f"L3 block {p} was written under another cache layout or with other weights")
                buf = memoryview(self.staging.numpy())
                pos = 0
                while pos < self.block_nbytes:
                    got = os.preadv(fd, [buf[pos:]], len(self.header) + pos)
                    if got <= 0:
                        raise ValueError(f"L3 block {p} is truncated")
                    pos += got
            finally:
                os.close(fd)
            off = 0
            for v, n in zip(self.views(bid), self.segments):
                src = self.staging[off:off + n].to(v.device, non_blocking=True)
                v.copy_(src.view(v.dtype).reshape(v.shape))
                off += n
            if self.cache.device.type == "cuda":
                torch.cuda.current_stream().synchronize()      # the staging buffer is reused by the next block
            self.index.lookup(h)                               # refresh LRU position
            self.bytes_loaded += self.block_nbytes
            self.n_load += 1
            self.t_load += time.monotonic() - t0
            n_ok += 1
        return n_ok

    def stats(self) -> dict:
        def bw(b, t):
            return b / t / (1 << 30) if t > 0 else 0.0
        return {"blocks": len(self), "n_store": self.n_store, "n_load": self.n_load, "n_evicted": self.n_evicted,
                "GiB_stored": self.bytes_stored / (1 << 30), "GiB_loaded": self.bytes_loaded / (1 << 30),
                "store_GiBps": bw(self.bytes_stored, self.t_store), "load_GiBps": bw(self.bytes_loaded, self.t_load)}

    def close(self):
        self.staging = None


def prompt_block_hashes(token_ids: Sequence[int], block_size: int) -> List[int]:
    """Chained hashes of the full blocks of a prompt that the prefix cache may serve (at most len-1 tokens are cached)."""
    out, h = [], 0
    for b in range((len(token_ids) - 1) // block_size):
        h = C.chain_hash(h, list(token_ids[b * block_size:(b + 1) * block_size]))
        out.append(h)
    return out
