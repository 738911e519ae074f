"""The allocation-free batch copy, called the way an embedding engine would call it: through the C symbol of the shared
library, with plain integer addresses. Such engines own all device memory themselves, so the library must not ask the
driver for any; this test checks that the entry point produces exactly the bytes the regular batch copy produces, on two
calls in a row (the second call reuses the built-in table area that the first one filled).

The file name sorts last on purpose: if this addition ever breaks, a run that stops at the first failure has already
exercised everything else."""
import ctypes
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "memfabric_hybrid_b200", "lib", "libmf_core.so")


def _entry():
    lib = ctypes.CDLL(LIB)
    fn = lib.mf_batch_xcopy_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.POINTER(ctypes.c_uint64), ctypes.POINTER(ctypes.c_uint64), ctypes.POINTER(ctypes.c_uint64), ctypes.c_uint32, ctypes.c_void_p]
    return fn


def _arr(values):
    return (ctypes.c_uint64 * len(values))(*values)


def _layout(count, region, rng):
    slot = region // count // 64 * 64
    sizes = [int(rng.integers(1, slot - 32)) for _ in range(count)]
    soffs = [i * slot + int(rng.integers(0, 16)) for i in range(count)]
    doffs = [i * slot + int(rng.integers(0, 16)) for i in range(count)]
    return sizes, soffs, doffs


def test_matches_regular_batch_copy_twice(mf):
    import torch

    torch.cuda.set_device(0)
    fn = _entry()
    region = 24 << 20
    src = torch.empty(region, dtype=torch.uint8, device="cuda")
    out_new = torch.empty(region, dtype=torch.uint8, device="cuda")
    out_old = torch.empty(region, dtype=torch.uint8, device="cuda")
    assert fn(None, None, None, 0, None) == 0  # warm-up: resolves the built-in table's address, launches nothing
    side = torch.cuda.Stream()
    for call, count in enumerate((150, 97)):  # within the regular entry point's inline limit so both paths can run it
        rng = np.random.default_rng(40 + call)
        src.copy_(torch.from_numpy(rng.integers(0, 256, region, dtype=np.uint8)).cuda())
        out_new.fill_(0x5A)
        out_old.fill_(0x5A)
        sizes, soffs, doffs = _layout(count, region, rng)
        srcs = [src.data_ptr() + o for o in soffs]
        # first call on the current stream, second on a stream of its own (ordered after the fills by the synchronize)
        stream = torch.cuda.current_stream().cuda_stream if call == 0 else side.cuda_stream
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        rc = fn(_arr(srcs), _arr([out_new.data_ptr() + o for o in doffs]), _arr(sizes), count, ctypes.c_void_p(stream))
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before, "the allocation-free entry point changed the amount of free device memory"
        assert mf.native.batch_xcopy_inline(srcs, [out_old.data_ptr() + o for o in doffs], sizes, 0, stream) == 0
        torch.cuda.synchronize()
        assert torch.equal(out_new, out_old), f"call {call}: the two entry points disagree"
        # and both are right: every block landed, nothing else was touched
        host_src, host_out = src.cpu().numpy(), out_new.cpu().numpy()
        expect = np.full(region, 0x5A, dtype=np.uint8)
        for s, d, n in zip(soffs, doffs, sizes):
            expect[d:d + n] = host_src[s:s + n]
        assert (host_out == expect).all()


def test_large_table_and_limits(mf):
    import torch

    torch.cuda.set_device(0)
    fn = _entry()
    # 3000 small copies: far beyond what fits in kernel parameters, still inside the fixed table
    count, blk = 3000, 4096
    src = torch.randint(0, 256, (count * blk,), dtype=torch.uint8, device="cuda")
    dst = torch.zeros(count * blk, dtype=torch.uint8, device="cuda")
    perm = np.random.default_rng(1).permutation(count)
    srcs = [src.data_ptr() + int(i) * blk for i in range(count)]
    dsts = [dst.data_ptr() + int(p) * blk for p in perm]
    assert fn(_arr(srcs), _arr(dsts), _arr([blk] * count), count, None) == 0
    torch.cuda.synchronize()
    assert torch.equal(dst.view(count, blk)[torch.from_numpy(perm).cuda()], src.view(count, blk))
    # limits are refused with a status, nothing is launched
    assert fn(_arr(srcs[:1] * 4097), _arr(dsts[:1] * 4097), _arr([blk] * 4097), 4097, None) == -3
    assert fn(_arr(srcs[:2]), _arr(dsts[:2]), _arr([1 << 31, 1 << 31]), 2, None) == -3  # 4 GiB of chunks > 2 GiB budget
    assert fn(_arr(srcs[:1]), _arr(dsts[:1]), _arr([0]), 1, None) == -2
    assert fn(None, None, None, 0, None) == 0
