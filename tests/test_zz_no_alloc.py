"""The allocation-free flash-decode entry point (for hosts that cannot call cudaMalloc, e.g. inside a foreign
stream capture or a process whose pool owns the whole device) must give the same output as the regular entry
point. It is called through its exported C symbol, twice in a row, because the built-in scratch keeps the
previous call's contents. This file sorts last on purpose: a failure here cannot hide other tests' results."""
import ctypes as C
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_static_scratch_entry_matches_regular_entry():
    from inferencehackathon_b200.ops import build, lib
    lib.load()
    raw = C.CDLL(build.KERNEL_LIB)                       # the exported symbols themselves
    fn = raw.ihb_flash_decode_static
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_void_p,
                   C.c_void_p]
    raw.ihb_flash_decode_static_error.restype = C.c_char_p
    raw.ihb_flash_decode_static_bytes.restype = C.c_size_t
    assert 0 < raw.ihb_flash_decode_static_bytes() <= 2 << 20
    d = torch.device("cuda", 0)
    g = torch.Generator(device=d).manual_seed(42)
    nq, nkv, max_seq, nsplit = 16, 2, 2048, 7
    kc = torch.randn(nkv, max_seq, 128, device=d, generator=g).to(torch.bfloat16)
    vc = torch.randn(nkv, max_seq, 128, device=d, generator=g).to(torch.bfloat16)
    stream = torch.cuda.current_stream().cuda_stream
    for ctx in (1500, 333):                              # two calls in a row on the same built-in scratch
        q = torch.randn(nq * 128, device=d, generator=g)
        pos = torch.tensor([ctx - 1], dtype=torch.int32, device=d)
        ref = torch.zeros(nq * 128, device=d)
        scratch = torch.zeros(lib.flash_decode_scratch_floats(nq, nsplit), device=d)
        ctrs = torch.zeros(nq, dtype=torch.int32, device=d)
        lib.flash_decode(q, kc, vc, nq, nkv, max_seq, pos, nsplit, scratch, ctrs, ref, False)
        out = torch.full((nq * 128,), float("nan"), device=d)
        rc = fn(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), nq, nkv, max_seq, pos.data_ptr(), nsplit, out.data_ptr(),
                stream)
        assert rc == 0, raw.ihb_flash_decode_static_error()
        torch.cuda.synchronize()
        assert float((out - ref).abs().max()) < 2e-3
        # and against plain PyTorch
        kf, vf = kc[:, :ctx].float(), vc[:, :ctx].float()
        sc = torch.einsum("kgd,ksd->kgs", q.reshape(nkv, nq // nkv, 128), kf) / math.sqrt(128)
        exp = torch.einsum("kgs,ksd->kgd", torch.softmax(sc, -1), vf).reshape(-1)
        assert float((out - exp).abs().max()) < 2e-3
    # a problem larger than the built-in scratch is refused with a message, nothing is launched
    rc = fn(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), nq, nkv, max_seq, pos.data_ptr(), 4096, out.data_ptr(), stream)
    assert rc != 0 and b"exceed" in raw.ihb_flash_decode_static_error()
    # so is a split count the kernel does not take although the scratch would hold it, and a head grouping it does not
    # support: each refusal names its reason
    rc = fn(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), 4, 2, max_seq, pos.data_ptr(), 512, out.data_ptr(), stream)
    assert rc != 0 and b"splits" in raw.ihb_flash_decode_static_error()
    rc = fn(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), 6, 2, max_seq, pos.data_ptr(), 4, out.data_ptr(), stream)
    assert rc != 0 and b"per KV head" in raw.ihb_flash_decode_static_error()
    rc = fn(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), 5, 2, max_seq, pos.data_ptr(), 4, out.data_ptr(), stream)
    assert rc != 0 and b"per KV head" in raw.ihb_flash_decode_static_error()
    torch.cuda.synchronize()
