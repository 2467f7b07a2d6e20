"""The non-allocating decode-attention entry point (``e2h_attn_decode_static``, declared in
``ops/csrc/attn_decode_static.h``) against the existing entry point with a caller-provided
scratch buffer. Collected last so that it also runs after every other GPU test has used the
library."""
import ctypes as C
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _symbol():
    from easy_to_hard_b200.ops import _lib
    fn = _lib.lib().e2h_attn_decode_static
    vp, i = C.c_void_p, C.c_int
    fn.argtypes = [vp, vp, vp, vp, vp, vp, i, i, i, i, i, C.c_float, i, vp]
    fn.restype = C.c_int
    return fn


def _case(B, n_head, n_kv, D, smax, pos, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.randn(B, n_head * D, device="cuda", generator=g).bfloat16()
    k = torch.randn(B, n_kv, smax, D, device="cuda", generator=g).bfloat16()
    v = torch.randn(B, n_kv, smax, D, device="cuda", generator=g).bfloat16()
    p = torch.tensor([pos], dtype=torch.int32, device="cuda")
    lp = torch.randint(0, max(1, pos // 4), (B,), device="cuda", generator=g).int()
    return q, k, v, p, lp


def _static(fn, q, k, v, p, lp, n_head, n_split, out=None):
    from easy_to_hard_b200.ops import _lib
    if out is None:
        out = torch.empty_like(q)
    B, n_kv, smax, D = q.shape[0], k.shape[1], k.shape[2], k.shape[3]
    rc = fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), p.data_ptr(),
            lp.data_ptr(), B, n_head, n_kv, D, smax, 1.0 / math.sqrt(D), n_split, _lib.stream())
    return rc, out


@pytest.mark.parametrize("B,n_head,n_kv,D,n_split", [(4, 32, 32, 128, 8), (3, 8, 2, 128, 4),
                                                      (8, 8, 8, 64, 2), (2, 4, 4, 128, 1)])
def test_static_scratch_matches_existing_entry(B, n_head, n_kv, D, n_split):
    from easy_to_hard_b200.ops import functional as Fn
    fn = _symbol()
    smax = 512
    # first call on the device: does the one-time address look-up (outside any capture)
    rc, first = _static(fn, *_case(B, n_head, n_kv, D, smax, 100, 0), n_head, n_split)
    assert rc == 0
    torch.cuda.synchronize()
    del first
    # two calls in a row, different inputs and lengths, sharing the array
    c1 = _case(B, n_head, n_kv, D, smax, 300, 1)
    c2 = _case(B, n_head, n_kv, D, smax, 37, 2)
    want1 = Fn.attn_decode(c1[0], c1[1], c1[2], c1[3], c1[4], n_head, n_split=n_split)
    want2 = Fn.attn_decode(c2[0], c2[1], c2[2], c2[3], c2[4], n_head, n_split=n_split)
    got1, got2 = torch.empty_like(want1), torch.empty_like(want2)
    torch.cuda.synchronize()
    alloc0, reserved0 = torch.cuda.memory_allocated(), torch.cuda.memory_reserved()
    free0 = torch.cuda.mem_get_info()[0]
    rc1 = _static(fn, *c1, n_head, n_split, out=got1)[0]
    rc2 = _static(fn, *c2, n_head, n_split, out=got2)[0]
    torch.cuda.synchronize()
    assert rc1 == 0 and rc2 == 0
    assert torch.equal(got1, want1)
    assert torch.equal(got2, want2)
    # nothing was allocated in between, by the caching allocator or behind its back
    assert torch.cuda.memory_allocated() == alloc0
    assert torch.cuda.memory_reserved() == reserved0
    assert torch.cuda.mem_get_info()[0] >= free0 - (2 << 20)


def test_static_scratch_refuses_beyond_limit():
    fn = _symbol()
    B, n_head, D, n_split = 64, 32, 128, 16        # twice the fixed array
    q, k, v, p, lp = _case(1, 1, 1, D, 16, 4, 3)   # never dereferenced: the call must not launch
    out = torch.zeros(4, device="cuda")
    rc = fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), p.data_ptr(), lp.data_ptr(),
            B, n_head, n_head, D, 16, 1.0, n_split, None)
    assert rc == -4
    torch.cuda.synchronize()
    assert float(out.abs().sum()) == 0.0
