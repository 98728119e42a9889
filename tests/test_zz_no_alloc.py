"""The allocation-free attention entry point, called through its exported C symbol.

Some users of the native library cannot allocate device memory when they need attention (inside a stream
capture, in a serving loop where cudaMalloc would stall the device, or under a fixed memory budget), so
`cuteafd_paged_attention_noalloc` keeps the split-KV scratch inside the library.  This test loads the shared
library with ctypes, calls that symbol directly twice in a row on different inputs (the built-in scratch keeps
the first call's contents, so the second call checks that stale partials are harmless) and compares each result
with the ordinary entry point, which gets caller-provided scratch.  It also checks that an oversized request is
refused with a clear message.  The file name sorts last so a run that stops at the first failure has already
exercised everything else.
"""
import ctypes as C

import pytest
import torch

from cuteafd_b200.ops import native

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _case(seed, Hq, Hkv, D, lens, qlens, n_pages=16):
    g = torch.Generator().manual_seed(seed)
    cache = torch.randn(n_pages * 64, 2, Hkv, D, generator=g).to(torch.bfloat16).to(DEV)
    perm = (torch.randperm(n_pages - 1, generator=g) + 1).tolist()
    pt = torch.zeros(len(lens), 8, dtype=torch.int32)
    p = 0
    for i, L in enumerate(lens):
        n = -(-L // 64)
        pt[i, :n] = torch.tensor(perm[p:p + n])
        p += n
    T = sum(qlens)
    q = torch.randn(T, Hq * D, generator=g).to(torch.bfloat16).to(DEV)
    q_start = torch.tensor([sum(qlens[:i]) for i in range(len(qlens))], dtype=torch.int32, device=DEV)
    return dict(q=q, kv=cache, pt=pt.to(DEV), kv_len=torch.tensor(lens, dtype=torch.int32, device=DEV), q_start=q_start,
                q_len=torch.tensor(qlens, dtype=torch.int32, device=DEV), T=T, n_seq=len(lens), max_q=max(qlens), Hq=Hq, Hkv=Hkv, D=D)


def _run(lib, c, splits, use_noalloc):
    out = torch.zeros(c["T"], c["Hq"] * c["D"], dtype=torch.bfloat16, device=DEV)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    P = lambda t: C.c_void_p(t.data_ptr())
    scale = C.c_float(c["D"] ** -0.5)
    if use_noalloc:
        fn = lib.cuteafd_paged_attention_noalloc
        fn.restype = C.c_int
        rc = fn(P(c["q"]), P(c["kv"]), P(c["pt"]), P(c["kv_len"]), P(c["q_start"]), P(c["q_len"]), None, P(out), c["T"], c["n_seq"],
                c["max_q"], c["Hq"] * c["D"], c["Hq"], c["Hkv"], c["D"], c["pt"].shape[1], splits, 0, scale, stream)
    else:
        po = torch.zeros(splits * c["T"] * c["Hq"] * c["D"], dtype=torch.float32, device=DEV)
        pml = torch.zeros(splits * c["T"] * c["Hq"] * 2, dtype=torch.float32, device=DEV)
        fn = lib.cuteafd_paged_attention
        fn.restype = C.c_int
        fn.argtypes = None
        rc = fn(P(c["q"]), P(c["kv"]), P(c["pt"]), P(c["kv_len"]), P(c["q_start"]), P(c["q_len"]), None, P(out), P(po), P(pml),
                c["T"], c["n_seq"], c["max_q"], c["Hq"] * c["D"], c["Hq"], c["Hkv"], c["D"], c["pt"].shape[1], splits, 0, scale, stream)
    torch.cuda.synchronize()
    return rc, out


def test_noalloc_entry_matches_regular_entry_twice_in_a_row():
    lib = C.CDLL(str(native.LIB_PATH))
    lib.cuteafd_last_error.restype = C.c_char_p
    cases = [(_case(1, 8, 2, 64, [200, 90, 7], [1, 3, 7]), 3), (_case(2, 16, 4, 128, [130, 64], [2, 1]), 2)]
    for c, splits in cases:                      # two calls in a row share the built-in scratch
        rc, got = _run(lib, c, splits, True)
        assert rc == 0, lib.cuteafd_last_error().decode()
        rc, want = _run(lib, c, splits, False)
        assert rc == 0, lib.cuteafd_last_error().decode()
        assert torch.allclose(got.float(), want.float(), atol=2e-2, rtol=2e-2)
        assert torch.isfinite(got.float()).all()


def test_noalloc_entry_refuses_oversized_requests():
    lib = C.CDLL(str(native.LIB_PATH))
    lib.cuteafd_last_error.restype = C.c_char_p
    c = _case(3, 16, 4, 128, [100], [1])
    big = dict(c)
    big["T"] = 4096                      # 32 splits x 4096 rows x 16 heads x 130 floats >> 2M floats
    rc, _ = _run(lib, dict(big, q=torch.zeros(4096, 16 * 128, dtype=torch.bfloat16, device=DEV)), 32, True)
    assert rc != 0 and b"scratch" in lib.cuteafd_last_error()
