"""Non-GEMM kernels (norm, embedding, decode attention, sampler) against PyTorch fp32 references."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _mk(*shape, scale=1.0, seed=0, dtype=torch.bfloat16):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, generator=g, device="cuda") * scale).to(dtype)


def _status_ok():
    from easy_to_hard_b200.ops import _lib
    torch.cuda.synchronize()
    assert _lib.read_status() == 0


@pytest.mark.parametrize("T,dim", [(64, 4096), (5, 256), (300, 1024)])
def test_rmsnorm(T, dim):
    from easy_to_hard_b200.ops import functional as Fn, reference
    x, w = _mk(T, dim, seed=1), _mk(dim, seed=2)
    y = Fn.rmsnorm(x, w, 1e-5)
    _status_ok()
    want = reference.rmsnorm(x, w, 1e-5)
    assert torch.allclose(y.float(), want.float(), rtol=2e-2, atol=2e-2)


def test_fused_residual_rmsnorm_with_partials_and_embedding():
    from easy_to_hard_b200.ops import functional as Fn, reference
    T, dim, V = 64, 512, 1000
    h, w = _mk(T, dim, seed=3), _mk(dim, seed=4)
    parts = _mk(4, T, dim, seed=5, dtype=torch.float32)
    h_out, x_out = torch.empty_like(h), torch.empty_like(h)
    Fn.fused_residual_rmsnorm(h, w, 1e-5, partials=parts, h_out=h_out, x_out=x_out)
    _status_ok()
    want_h = (h.float() + parts.sum(0).bfloat16().float()).bfloat16()
    assert torch.allclose(h_out.float(), want_h.float(), rtol=1e-2, atol=2e-2)
    assert torch.allclose(x_out.float(), reference.rmsnorm(want_h, w, 1e-5).float(), rtol=2e-2,
                          atol=3e-2)
    emb = _mk(V, dim, seed=6)
    tok = torch.randint(0, V, (T,), device="cuda", dtype=torch.int32)
    Fn.fused_residual_rmsnorm(None, w, 1e-5, tokens=tok, emb=emb, h_out=h_out, x_out=x_out)
    _status_ok()
    assert torch.equal(h_out, emb[tok.long()])
    assert torch.allclose(x_out.float(), reference.rmsnorm(emb[tok.long()], w, 1e-5).float(),
                          rtol=2e-2, atol=3e-2)
    assert torch.equal(Fn.embedding(tok.view(8, 8), emb), emb[tok.long()].view(8, 8, dim))


def test_rmsnorm_bwd_and_swiglu_bwd():
    from easy_to_hard_b200.ops import functional as Fn
    T, dim = 37, 512
    x, w, dy = _mk(T, dim, seed=7), _mk(dim, seed=8), _mk(T, dim, seed=9)
    xf = x.float().requires_grad_(True)
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * w.float()
    y.backward(dy.float())
    dx = Fn.rmsnorm_bwd(x, dy, w, 1e-5)
    assert torch.allclose(dx.float(), xf.grad, rtol=2e-2, atol=3e-2)
    g, u, d = _mk(T, dim, seed=10), _mk(T, dim, seed=11), _mk(T, dim, seed=12)
    gf, uf = g.float().requires_grad_(True), u.float().requires_grad_(True)
    (torch.nn.functional.silu(gf) * uf).backward(d.float())
    dg, du = Fn.swiglu_bwd(g, u, d)
    assert torch.allclose(dg.float(), gf.grad, rtol=2e-2, atol=3e-2)
    assert torch.allclose(du.float(), uf.grad, rtol=2e-2, atol=3e-2)
    assert torch.allclose(Fn.swiglu(g, u).float(), (torch.nn.functional.silu(g) * u).float(),
                          rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("B,n_head,n_kv,D,pos,n_split", [
    (64, 32, 32, 128, 300, 1), (3, 8, 2, 128, 77, 1), (2, 8, 8, 64, 40, 4), (1, 32, 8, 128, 500, 8),
    (5, 4, 1, 64, 0, 1), (4, 8, 1, 128, 33, 2),
    (600, 4, 1, 64, 70, 8)])        # more sequences than one launch takes: goes in slices
def test_attn_decode(B, n_head, n_kv, D, pos, n_split):
    from easy_to_hard_b200.ops import functional as Fn, reference
    smax = 512
    q = _mk(B, n_head * D, seed=13)
    kc, vc = _mk(B, n_kv, smax, D, seed=14), _mk(B, n_kv, smax, D, seed=15)
    left = torch.randint(0, max(pos // 2, 1), (B,), device="cuda", dtype=torch.int32)
    p = torch.tensor([pos], dtype=torch.int32, device="cuda")
    o = Fn.attn_decode(q, kc, vc, p, left, n_head, n_split=n_split)
    _status_ok()
    j = torch.arange(smax, device="cuda")
    mask = (j[None] <= pos) & (j[None] >= left[:, None])
    want = reference.attention(q.view(B, n_head, 1, D), kc, vc, mask[:, None, None, :])
    assert torch.allclose(o.view(B, n_head, 1, D).float(), want.float(), rtol=2e-2, atol=2e-2)


def test_attn_decode_shared_pairs_merge_in_kernel_and_replay():
    """(sequence, kv head) pairs cut by the CTAs' run boundaries are merged by the last of their
    CTAs to finish: close to the one-CTA-per-pair form, bit-identical from call to call
    (the parts are combined in CTA order), and the ticket words return to zero, so later calls
    (and graph replays) need no reset. Long contexts with few pairs force up to 8 parts."""
    from easy_to_hard_b200.ops import functional as Fn
    for B, n_head, n_kv, D, smax, pos in [(6, 8, 2, 128, 512, 411), (2, 32, 32, 128, 4096, 4001),
                                          (64, 32, 32, 128, 640, 607), (9, 32, 8, 128, 300, 290)]:
        q = _mk(B, n_head * D, seed=31)
        kc, vc = _mk(B, n_kv, smax, D, seed=32), _mk(B, n_kv, smax, D, seed=33)
        left = torch.randint(0, pos // 3, (B,), device="cuda", dtype=torch.int32)
        p = torch.tensor([pos], dtype=torch.int32, device="cuda")
        whole = Fn.attn_decode(q, kc, vc, p, left, n_head, n_split=1)
        first = Fn.attn_decode(q, kc, vc, p, left, n_head, n_split=8)
        assert torch.allclose(first.float(), whole.float(), rtol=2e-2, atol=2e-2)
        for n_split in (8, 2, 0):
            again = Fn.attn_decode(q, kc, vc, p, left, n_head, n_split=n_split)
            if n_split in (8, 0):
                assert torch.equal(again, first)
            else:
                assert torch.allclose(again.float(), whole.float(), rtol=2e-2, atol=2e-2)
    _status_ok()


@pytest.mark.parametrize("top_k,ties", [(50, False), (1, False), (256, False), (300, False),
                                        (50, True), (3, True)])
def test_sampler_pivot_paths_keep_exactly_the_top_k(top_k, ties):
    """The top-k pivot comes from the candidate path (row in shared memory, k <= 256), from
    the radix select (k > 256) or from the radix select as the fall-back (more entries tie at
    the bound than the candidate list holds): in every case a draw is one of the entries
    whose value is at least the k-th largest, and over many draws all of them turn up."""
    from easy_to_hard_b200.ops import functional as Fn
    B, V = 32, 32016
    g = torch.Generator(device="cuda").manual_seed(77)
    row = torch.randn(V, device="cuda", generator=g) * 2
    if ties:
        row[torch.randperm(V, device="cuda", generator=g)[:6000]] = 7.5   # 6000 equal maxima
    logits = row[None].expand(B, V).contiguous()
    kth = row.topk(top_k).values[-1]
    allowed = row >= kth                      # ties with the pivot are kept, as the reference does
    pos = torch.zeros(1, dtype=torch.int32, device="cuda")
    nxt = torch.zeros(B, dtype=torch.int32, device="cuda")
    seen = torch.zeros(V, dtype=torch.bool, device="cuda")
    for it in range(40 if allowed.sum() < 400 else 8):
        pos.fill_(it)
        Fn.sample(logits, temperature=1.5, top_k=top_k, seed=99, pos=pos, next_tok=nxt,
                  advance_pos=False)
        assert allowed[nxt.long()].all()
        seen[nxt.long()] = True
    if int(allowed.sum()) <= 50:
        assert int(seen.sum()) >= min(int(allowed.sum()), 20)
    _status_ok()


def test_sampler_greedy_topk_and_bookkeeping():
    from easy_to_hard_b200.ops import functional as Fn
    B, V = 16, 32016
    logits = _mk(B, V, seed=16, dtype=torch.float32) * 3
    pos = torch.tensor([9], dtype=torch.int32, device="cuda")
    nxt = torch.zeros(B, dtype=torch.int32, device="cuda")
    seq = torch.zeros(B, 32, dtype=torch.int32, device="cuda")
    eos = torch.zeros(B, dtype=torch.int32, device="cuda")
    ticket = torch.zeros(1, dtype=torch.int32, device="cuda")
    Fn.sample(logits, temperature=0.0, top_k=None, seed=1, pos=pos, next_tok=nxt, seq=seq,
              eos_id=int(logits[0].argmax()), eos_flag=eos, ticket=ticket)
    assert torch.equal(nxt.long(), logits.argmax(-1))
    assert pos.item() == 10 and torch.equal(seq[:, 10], nxt) and eos[0].item() == 1
    # top-k sampling: every draw lies in the top-k set, and frequencies follow softmax(top-k)
    k, temp, n = 5, 0.7, 4000
    row = logits[:1].expand(B, V).contiguous()
    topv, topi = row[0].topk(k)
    want = torch.softmax(topv / temp, -1)
    counts = torch.zeros(k, device="cuda")
    for it in range(n // B):
        pos.fill_(it)
        Fn.sample(row, temperature=temp, top_k=k, seed=1234, pos=pos, next_tok=nxt,
                  advance_pos=False)
        hit = nxt.long()[:, None] == topi[None]
        assert hit.any(-1).all()
        counts += hit.float().sum(0)
    freq = counts / counts.sum()
    assert (freq - want).abs().max().item() < 0.04
