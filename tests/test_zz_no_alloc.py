"""The allocation-free top-k encoder, called through its exported C symbol.

Some users of the library cannot allocate device memory at the point where they
compress a gradient (a frozen memory pool, an allocator callback, a GPU whose
memory another allocator already owns).  ``hp_cuda_sparse_encode_noalloc`` serves
them with scratch that lives inside the library.  This file checks it against the
ordinary entry point (which takes caller-allocated scratch) on two calls in a row,
because the shared scratch keeps the first call's contents when the second starts.
It is named to be collected last so that a run stopping at the first failure has
already run everything else."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from hipress_b200._native import lib
    L = lib.cuda()  # same shared object the package uses; the symbol is looked up by name
    fn = L.hp_cuda_sparse_encode_noalloc
    fn.restype = C.c_int
    fn.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint64,
                   C.c_uint64, C.c_float, C.c_int, C.c_void_p, C.c_int, C.c_void_p]
    L.hp_cuda_noalloc_scratch_bytes.restype = C.c_uint64
    return lib, L, fn


def _pairs(payload, kmax):
    from hipress_b200.ops import sparse_pairs
    return sparse_pairs(payload, kmax)


@pytest.mark.parametrize("alg_name,alg", [("dgc", 4), ("graddrop", 5)])
def test_noalloc_matches_regular_entry_point_twice(alg_name, alg):
    lib, L, fn = _lib()
    from hipress_b200.ops import Compressor
    comp = Compressor(alg_name, ratio=0.001)
    n = 1_000_003
    k = comp.kmax(n)
    nbytes = comp.payload_bytes(n)
    torch.manual_seed(5)
    st_a = comp.new_state(n, "cuda")          # state driven through the regular entry point
    st_b = {k_: v.clone() for k_, v in st_a.items()}  # state driven through the new one
    ws = comp.new_workspace("cuda", n)
    stream = lib.stream_ptr()
    for call in range(2):                      # two calls in a row share the internal scratch
        g = torch.randn(n, device="cuda")
        pa = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
        pb = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
        comp.encode(g, st_a, out=pa, workspace=ws)
        acc = st_b["accum_v"] if alg_name == "dgc" else st_b["residual"]
        u = st_b.get("momentum_u")
        rc = fn(alg, g.data_ptr(), acc.data_ptr(), None if u is None else u.data_ptr(), n, k, k,
                comp.spec.momentum, 1, pb.data_ptr(), 0, stream)
        assert rc == 0, lib.cuda().hp_cuda_error_string(rc)
        torch.cuda.synchronize()
        ia, va = _pairs(pa, k)
        ib, vb = _pairs(pb, k)
        assert ia.numel() == k
        assert torch.equal(ia, ib), f"call {call}: different elements selected"
        assert torch.allclose(va, vb, rtol=1e-6, atol=0), f"call {call}: values differ"
        assert torch.equal(pa[:16].cpu(), pb[:16].cpu()), "headers differ"
        for name in st_a:
            assert torch.allclose(st_a[name], st_b[name], rtol=1e-6, atol=1e-9), name


def test_noalloc_rejects_oversized_input_and_reports_scratch_size():
    lib, L, fn = _lib()
    too_many = (1 << 28) + 1
    dummy = torch.zeros(16, device="cuda")
    out = torch.zeros(64, dtype=torch.uint8, device="cuda")
    rc = fn(5, dummy.data_ptr(), dummy.data_ptr(), None, too_many, 1, 1, 0.9, 1, out.data_ptr(), 0,
            lib.stream_ptr())
    assert rc == -2  # HP_ERR_TOO_LARGE, nothing launched
    assert b"larger" in L.hp_cuda_error_string(rc)
    assert 0 < L.hp_cuda_noalloc_scratch_bytes() <= 64 * 1024
    torch.cuda.synchronize()
