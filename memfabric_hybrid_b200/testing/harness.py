"""Scripted multi-rank harness: N rank processes that execute commands sent by one driver.

The driver (a test, a notebook, a debugging session) starts `RankHarness(world)`, then tells ranks what to do, one command at
a time or all ranks at once, and gets every command's result back:

    with RankHarness(2, gpus=[0, 1]) as h:
        h.all("bm_init", url, 2)                 # every rank, in parallel; returns [result of rank 0, result of rank 1]
        h.all("bm_create", hbm_bytes, dram_bytes)
        h.all("bm_join")
        buf = h.call(0, "alloc", "host_pinned", 64 << 20)      # a named local buffer on rank 0
        h.call(0, "fill", buf, 0, 64 << 20, 1234)
        h.call(0, "copy", buf, ("hbm", 1, 0), 64 << 20)        # rank 0's buffer -> rank 1's pooled HBM, offset 0
        assert h.call(1, "checksum", ("hbm", 1, 0), 64 << 20) == h.call(0, "checksum", buf, 64 << 20)

A location is either the name of a local buffer (optionally `(name, offset)`) or a pool address `(kind, rank, offset)` with
kind "hbm" or "dram". Commands raise in the rank and the exception text comes back as `HarnessError` in the driver, so a test
reads like a script and fails at the line that went wrong. Same role as the reference's command server for multi-process tests
(test/python/mock_server/server.py:62-240 command loop, :527-960 command set), with pipes instead of sockets.
"""
from __future__ import annotations

import multiprocessing as mp
import os
import traceback
from typing import Any, Sequence


class HarnessError(RuntimeError):
    pass


def _rank_main(rank: int, world: int, conn, gpu, env):
    for k, v in (env or {}).items():
        os.environ[k] = str(v)
    state: dict[str, Any] = {"rank": rank, "world": world, "gpu": gpu, "bufs": {}, "keep": []}
    try:
        import memfabric_hybrid_b200 as mf

        state["mf"] = mf
        if gpu is not None:
            import torch

            torch.cuda.set_device(gpu)
            state["torch"] = torch
    except Exception:  # pragma: no cover - reported on the first command
        state["import_error"] = traceback.format_exc()
    while True:
        try:
            msg = conn.recv()
        except EOFError:
            break
        if msg is None:
            break
        name, args = msg
        try:
            if "import_error" in state:
                raise RuntimeError(state["import_error"])
            fn = _COMMANDS.get(name)
            if fn is None:
                raise KeyError(f"unknown command {name!r}")
            conn.send(("ok", fn(state, *args)))
        except Exception as ex:  # noqa: BLE001
            conn.send(("err", f"rank {rank}: {name}{args!r}: {ex!r}\n{traceback.format_exc()}"))
    try:
        _cmd_shutdown(state)
    except Exception:  # noqa: BLE001
        pass


# ---------------------------------------------------------------------------------------------------------- commands

def _addr(state, loc) -> int:
    """Location → address. str | (str, off): a local buffer; (kind, rank, off): pooled memory."""
    if isinstance(loc, int):
        return loc
    if isinstance(loc, str):
        return state["bufs"][loc]["addr"]
    if len(loc) == 2:
        return state["bufs"][loc[0]]["addr"] + int(loc[1])
    kind, rank, off = loc
    mf = state["mf"]
    mem = mf.bm.BmMemType.DEVICE if kind == "hbm" else mf.bm.BmMemType.HOST
    return state["bm"].peer_rank_ptr(mem, int(rank)) + int(off)


def _is_device(state, loc) -> bool:
    if isinstance(loc, (str, tuple)) and not (isinstance(loc, tuple) and len(loc) == 3):
        name = loc if isinstance(loc, str) else loc[0]
        return state["bufs"][name]["kind"] == "device"
    return isinstance(loc, tuple) and loc[0] == "hbm"


def _cmd_ping(state):
    return {"rank": state["rank"], "pid": os.getpid(), "gpu": state["gpu"]}


def _cmd_setenv(state, key, value):
    os.environ[key] = str(value)


def _cmd_bm_init(state, url, world, auto_ranking=False, timeout=60):
    mf = state["mf"]
    cfg = mf.bm.BmConfig()
    cfg.auto_ranking = auto_ranking
    if not auto_ranking:
        cfg.rank_id = state["rank"]
    cfg.init_timeout = cfg.create_timeout = cfg.operation_timeout = timeout
    dev = state["gpu"] if state["gpu"] is not None else -1
    rc = mf.bm.initialize(url, world, dev, cfg)
    if rc != 0:
        raise RuntimeError(f"bm.initialize -> {rc}: {mf.get_last_err_msg()}")
    return mf.bm.bm_rank_id() if hasattr(mf.bm, "bm_rank_id") else state["rank"]


def _cmd_bm_create(state, hbm_bytes, dram_bytes, data_op=None):
    mf = state["mf"]
    if data_op is None:
        op = mf.bm.BmDataOpType.SDMA if state["gpu"] is not None else mf.bm.BmDataOpType.HOST_RDMA
    else:
        op = data_op
    # DRAM slices of GPU ranks go to the GPU's own NUMA node (flag bits 0-6 = 0x7F)
    flags = 0x7F if state["gpu"] is not None and dram_bytes > 0 else 0
    state["bm"] = mf.bm.create(0, dram_bytes, hbm_bytes if state["gpu"] is not None else 0, op, flags, dram_bytes, hbm_bytes)
    return True


def _cmd_bm_join(state):
    rc = state["bm"].join()
    if rc != 0:
        raise RuntimeError(f"join -> {rc}: {state['mf'].get_last_err_msg()}")
    return state["bm"].joined_size()


def _cmd_bm_leave(state):
    return state["bm"].leave()


def _cmd_joined_size(state):
    return state["bm"].joined_size()


def _cmd_ptr(state, kind, rank):
    return _addr(state, (kind, rank, 0))


def _cmd_alloc(state, kind, nbytes, name=None):
    """kind: host_pageable | host_pinned | device. Returns the buffer's name."""
    import numpy as np

    name = name or f"buf{len(state['bufs'])}"
    if kind == "host_pageable":
        a = np.zeros(nbytes, dtype=np.uint8)
        state["bufs"][name] = {"kind": "host", "addr": a.ctypes.data, "obj": a, "nbytes": nbytes}
    elif kind == "host_pinned":
        if state["gpu"] is not None:
            t = state["torch"].zeros(nbytes, dtype=state["torch"].uint8).pin_memory()
            state["bufs"][name] = {"kind": "host", "addr": t.data_ptr(), "obj": t, "nbytes": nbytes}
        else:
            a = np.zeros(nbytes, dtype=np.uint8)
            state["bufs"][name] = {"kind": "host", "addr": a.ctypes.data, "obj": a, "nbytes": nbytes}
    elif kind == "device":
        t = state["torch"].zeros(nbytes, dtype=state["torch"].uint8, device="cuda")
        state["bufs"][name] = {"kind": "device", "addr": t.data_ptr(), "obj": t, "nbytes": nbytes}
    else:
        raise ValueError(kind)
    return name


def _cmd_free(state, name):
    state["bufs"].pop(name, None)


def _cmd_fill(state, loc, nbytes, seed):
    """Writes the library's seeded byte pattern (the same function on host and device)."""
    mf, addr = state["mf"], _addr(state, loc)
    if _is_device(state, loc):
        s = state["torch"].cuda.current_stream().cuda_stream
        rc = mf.native.fill_pattern(addr, nbytes, seed, s)
        state["torch"].cuda.synchronize()
        if rc != 0:
            raise RuntimeError(f"fill_pattern -> {rc}")
    else:
        step = 8 << 20
        for off in range(0, nbytes, step):
            n = min(step, nbytes - off)
            mf.native.host_write(addr + off, mf.native.pattern_bytes(seed, off, n))
    return True


def _cmd_checksum(state, loc, nbytes):
    """Order-sensitive 64-bit checksum of the bytes, the same function on host and device."""
    mf, addr = state["mf"], _addr(state, loc)
    if _is_device(state, loc):
        torch = state["torch"]
        out = torch.zeros(1, dtype=torch.int64, device="cuda")
        rc = mf.native.checksum(addr, nbytes, out.data_ptr(), torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        if rc != 0:
            raise RuntimeError(f"checksum -> {rc}")
        return int(out.item()) & 0xFFFFFFFFFFFFFFFF
    return int(mf.native.checksum_host(mf.native.host_read(addr, nbytes))) & 0xFFFFFFFFFFFFFFFF


def _cmd_read(state, loc, nbytes):
    if _is_device(state, loc):
        torch = state["torch"]
        tmp = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
        mf = state["mf"]
        rc = mf.native.copy_engine(tmp.data_ptr(), _addr(state, loc), nbytes, torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        if rc != 0:
            raise RuntimeError(f"copy_engine -> {rc}")
        return bytes(tmp.numpy().tobytes())
    return state["mf"].native.host_read(_addr(state, loc), nbytes)


def _cmd_copy(state, src, dst, nbytes, copy_type=None, flags=0, expect_ok=True):
    mf = state["mf"]
    t = mf.bm.BmCopyType.AUTO if copy_type is None else getattr(mf.bm.BmCopyType, copy_type)
    rc = state["bm"].copy_data(_addr(state, src), _addr(state, dst), nbytes, t, flags)
    if rc != 0 and expect_ok:
        raise RuntimeError(f"copy_data -> {rc}: {mf.get_last_err_msg()}")
    if state["gpu"] is not None:
        state["bm"].wait()
        state["torch"].cuda.synchronize()
    return rc


def _cmd_copy_batch(state, srcs: Sequence, dsts: Sequence, sizes: Sequence[int], copy_type=None, flags=0, expect_ok=True):
    mf = state["mf"]
    t = mf.bm.BmCopyType.AUTO if copy_type is None else getattr(mf.bm.BmCopyType, copy_type)
    rc = state["bm"].copy_data_batch([_addr(state, s) for s in srcs], [_addr(state, d) for d in dsts], list(sizes), len(sizes), t, flags)
    if rc != 0 and expect_ok:
        raise RuntimeError(f"copy_data_batch -> {rc}: {mf.get_last_err_msg()}")
    if state["gpu"] is not None:
        state["bm"].wait()
        state["torch"].cuda.synchronize()
    return rc


def _cmd_stats(state):
    return dict(state["mf"].native.data_op_stats())


def _cmd_last_error(state):
    return state["mf"].get_last_err_msg()


def _cmd_eval(state, source):
    """Escape hatch for one-off scripts: evaluates an expression with `mf`, `state` and `addr` in scope."""
    return eval(source, {"mf": state["mf"], "state": state, "addr": lambda loc: _addr(state, loc)})  # noqa: S307


def _cmd_shutdown(state):
    state["bufs"].clear()
    bm = state.pop("bm", None)
    if bm is not None:
        bm.destroy()
        state["mf"].bm.uninitialize()
    return True


_COMMANDS = {
    "ping": _cmd_ping, "setenv": _cmd_setenv, "bm_init": _cmd_bm_init, "bm_create": _cmd_bm_create, "bm_join": _cmd_bm_join,
    "bm_leave": _cmd_bm_leave, "joined_size": _cmd_joined_size, "ptr": _cmd_ptr, "alloc": _cmd_alloc, "free": _cmd_free,
    "fill": _cmd_fill, "checksum": _cmd_checksum, "read": _cmd_read, "copy": _cmd_copy, "copy_batch": _cmd_copy_batch,
    "stats": _cmd_stats, "last_error": _cmd_last_error, "eval": _cmd_eval, "shutdown": _cmd_shutdown,
}


# ------------------------------------------------------------------------------------------------------------ driver

class RankHarness:
    """Starts `world` rank processes (spawned, so each has its own CUDA context) and relays commands to them.

    gpus: one device index per rank (None = CPU-only ranks). env: extra environment for every rank, or a list with one
    dict per rank (e.g. different MF_HOST_IDENTITY values to emulate several hosts)."""

    def __init__(self, world: int, gpus: Sequence[int] | None = None, env: dict | Sequence[dict] | None = None, timeout: float = 300.0):
        ctx = mp.get_context("spawn")
        self.world, self.timeout = world, timeout
        self._conns, self._procs = [], []
        for r in range(world):
            parent, child = ctx.Pipe()
            e = env[r] if isinstance(env, (list, tuple)) else env
            p = ctx.Process(target=_rank_main, args=(r, world, child, None if gpus is None else gpus[r], e), daemon=True)
            p.start()
            child.close()
            self._conns.append(parent)
            self._procs.append(p)

    def _send(self, rank, name, args):
        self._conns[rank].send((name, args))

    def _recv(self, rank):
        if not self._conns[rank].poll(self.timeout):
            raise HarnessError(f"rank {rank} did not answer within {self.timeout} s")
        try:
            status, value = self._conns[rank].recv()
        except EOFError:
            raise HarnessError(f"rank {rank} exited (exit code {self._procs[rank].exitcode})") from None
        if status != "ok":
            raise HarnessError(value)
        return value

    def call(self, rank: int, name: str, *args):
        """Runs one command on one rank and returns its result."""
        self._send(rank, name, args)
        return self._recv(rank)

    def all(self, name: str, *args, ranks: Sequence[int] | None = None):
        """Issues the command to every rank (or `ranks`) at once, then collects the results in rank order. Collective steps
        (join, barriers inside the library) need this form: the ranks must run them at the same time."""
        ranks = list(range(self.world)) if ranks is None else list(ranks)
        for r in ranks:
            self._send(r, name, args)
        errors, results = [], []
        for r in ranks:
            try:
                results.append(self._recv(r))
            except HarnessError as ex:
                errors.append(str(ex))
                results.append(None)
        if errors:
            raise HarnessError("\n".join(errors))
        return results

    def kill(self, rank: int):
        """Ends a rank abruptly (for failure-detection scenarios): the process is terminated between commands, so none of
        its work is in flight."""
        self._procs[rank].terminate()
        self._procs[rank].join(10)

    def close(self):
        for r, c in enumerate(self._conns):
            try:
                if self._procs[r].is_alive():
                    c.send(None)
            except (OSError, ValueError):
                pass
        for p in self._procs:
            p.join(30)
            if p.is_alive():
                p.terminate()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False
