"""Each mechanism of the Vomotar parts alone: its kernels against the plain function of the same
name in ``plain_vomotar``, at sizes that are no multiple of anything, with states carried from one
call to the next, and with inputs made so that a key one position outside a chunk, a far token in
a state or a lost convolution input would show."""

from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_vomotar as pv
from gpu_helpers import assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _ctx(seq_lens, pos0, slots):
    """The device arrays of a step of these sequences."""
    lens = np.asarray(seq_lens, dtype=np.int32)
    qstart = (np.cumsum(lens) - lens).astype(np.int32)
    token_seq = np.repeat(np.arange(len(lens), dtype=np.int32), lens)
    pos0 = np.asarray(pos0, dtype=np.int32)
    slots = np.asarray(slots, dtype=np.int32)
    positions = pos0[token_seq] + (np.arange(lens.sum(), dtype=np.int32) - qstart[token_seq])
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(DEV)
    host = SimpleNamespace(seq_qlen=lens, seq_pos0=pos0, seq_slot=slots, seq_qstart=qstart)
    return SimpleNamespace(n_seqs=len(lens), n_tokens=int(lens.sum()), token_seq=dev(token_seq),
                           token_slot=dev(slots[token_seq]), positions=dev(positions),
                           seq_slot=dev(slots), seq_qstart=dev(qstart), seq_qlen=dev(lens),
                           seq_pos0=dev(pos0), host=host,
                           status=torch.zeros(1, dtype=torch.int32, device=DEV))


def _gen(seed):
    return torch.Generator().manual_seed(seed)


@pytest.mark.parametrize("groups,width", [(1, 40), (2, 96), (5, 60), (16, 256)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_grouped_rms_norm(groups, width, dtype):
    from distengine_b200.kernels import ops
    g = _gen(groups)
    resid = torch.randn(7, width, generator=g) * 3
    delta = torch.randn(7, width, generator=g).to(dtype)
    weight = (torch.rand(width, generator=g) + 0.5).to(dtype)
    want = pv.grouped_rms_norm((resid + delta.float()).double(), weight.double(), groups, 1e-5)
    r = resid.to(DEV)
    out = torch.empty(7, width, dtype=dtype, device=DEV)
    ops.add_rmsnorm(r, delta.to(DEV), weight.to(DEV), 1e-5, out, groups=groups)
    assert_close(out, want, dtype, "grouped norm")
    assert_close(r, resid + delta.float(), torch.float32, "residual sum")
    rows = torch.tensor([5, 0, 5], dtype=torch.int32, device=DEV)
    picked = torch.empty(3, width, dtype=dtype, device=DEV)
    ops.add_rmsnorm(r, None, weight.to(DEV), 1e-5, picked, rows, groups=groups)
    assert_close(picked, want[[5, 0, 5]], dtype, "grouped norm of picked rows")


def _scan_inputs(T, H, G, dk, dv, seed):
    g = _gen(seed)
    q = pv.unit(torch.randn(T, G, dk, generator=g)) * dk ** -0.5
    k = pv.unit(torch.randn(T, G, dk, generator=g))
    v = torch.randn(T, H, dv, generator=g)
    beta = torch.sigmoid(torch.randn(T, H, generator=g))
    dec = torch.exp(-torch.rand(T, H, dk, generator=g) * 0.3)
    return q, k, v, beta, dec


@pytest.mark.parametrize("H,G,dk,dv", [(4, 2, 16, 24), (1, 1, 68, 33), (3, 3, 5, 130), (2, 1, 256, 16)])
def test_delta_rule_scan_carries_its_state(H, G, dk, dv):
    """Two sequences in unequal pieces over three calls, in slots 3 and 1 of 5; the state of an
    untouched slot stays as it is."""
    from distengine_b200.kernels import recurrent as rk
    lens = (37, 20)
    data = [_scan_inputs(n, H, G, dk, dv, 10 + i) for i, n in enumerate(lens)]
    rep = H // G
    want = [pv.gated_delta_rule(q.double().repeat_interleave(rep, 1),
                                k.double().repeat_interleave(rep, 1), v.double(), b.double(),
                                d.double()) for q, k, v, b, d in data]
    extra = 11                                          # the row is longer than the matrices
    state = torch.zeros(5, H * dk * dv + extra, device=DEV)
    state[2] = 7.0
    slots, fed = (3, 1), [0, 0]
    got = [torch.zeros(n, H, dv) for n in lens]
    for pieces in ((30, 1), (1, 17), (6, 2)):
        ctx = _ctx(pieces, fed, slots)
        cut = lambda i, j: torch.cat([data[s][i][fed[s]: fed[s] + pieces[s]].reshape(pieces[s], -1)
                                      for s in range(2)]).to(DEV).contiguous()
        n = sum(pieces)
        out = torch.empty(n, H * dv, device=DEV)
        rk.state_scan(cut(0, 0), cut(1, 0), cut(2, 0), state, out, H, G, dk, dv, ctx,
                      g=cut(4, 0), beta=cut(3, 0))
        at = 0
        for s in range(2):
            got[s][fed[s]: fed[s] + pieces[s]] = out[at: at + pieces[s]].cpu().view(-1, H, dv)
            at += pieces[s]
            fed[s] += pieces[s]
    for s in range(2):
        assert_close(got[s], want[s], torch.float32, f"delta rule, sequence {s}")
    assert bool((state[2] == 7.0).all()) and bool((state[0] == 0).all())
    assert bool((state[3, H * dk * dv:] == 0).all())


def test_retention_keeps_a_far_token():
    """No decay (1.0) and a query that points at the first token's key: 300 tokens later the
    read-out is that token's value; with decay 0.5 it is gone.  The values are bfloat16 rows of a
    wider matrix, as the mixer passes them."""
    from distengine_b200.kernels import recurrent as rk
    T, H, dk, dv = 301, 2, 12, 40
    g = _gen(3)
    k = torch.randn(T, H, dk, generator=g) * 0.01
    q = torch.randn(T, H, dk, generator=g) * 0.05
    v = torch.randn(T, H, dv, generator=g).to(torch.bfloat16)
    k[0] = 0
    k[0, :, 3] = 4.0
    q[300] = 0
    q[300, :, 3] = 4.0
    decay = torch.tensor([1.0, 0.5])
    want = pv.retention(q.double(), k.double(), v.double(), decay.double())
    first = 16 * v[0].double()
    assert (want[300, 0] - first[0]).abs().max() < 0.2 * first[0].abs().max()
    assert want[300, 1].abs().max() < 0.2 * first[1].abs().max()
    state = torch.zeros(2, H * dk * dv, device=DEV)
    wide = torch.zeros(T, 8 + H * dv, dtype=torch.bfloat16, device=DEV)
    wide[:, 8:] = v.reshape(T, -1).to(DEV)
    got = torch.empty(T, H * dv, device=DEV)
    at = 0
    for piece in (1, 2, 250, 47, 1):                    # prompt portions and single tokens
        ctx = _ctx((piece,), (at,), (1,))
        out = torch.empty(piece, H * dv, device=DEV)
        rk.state_scan(q[at: at + piece].reshape(piece, -1).to(DEV).contiguous(),
                      k[at: at + piece].reshape(piece, -1).to(DEV).contiguous(),
                      wide[at: at + piece, 8:], state, out, H, H, dk, dv, ctx, decay=decay.to(DEV))
        got[at: at + piece] = out
        at += piece
    assert_close(got.view(T, H, dv), want, torch.float32, "retention")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dims,dk", [(8, 8), (6, 20), (0, 4)])
def test_retention_rotation(dtype, dims, dk):
    from distengine_b200.kernels import recurrent as rk
    T, H = 9, 3
    g = _gen(dims)
    proj = torch.randn(T, 2 * H * dk + 5, generator=g).to(dtype)
    base = 50.0
    ctx = _ctx((4, 5), (1000, 3), (0, 1))
    pos = ctx.positions.cpu().numpy()
    inv = torch.tensor([base ** (-2.0 * i / max(dims, 1)) for i in range(dims // 2)],
                       dtype=torch.float32).to(DEV)
    qr = torch.empty(T, H * dk, device=DEV)
    kr = torch.empty(T, H * dk, device=DEV)
    rk.retention_prep(proj.to(DEV), inv, dims, H, dk, qr, kr, ctx)
    for n in range(T):                                  # the plain rotation at the token's position
        for which, got in ((0, qr), (1, kr)):
            x = proj[n, which * H * dk: (which + 1) * H * dk].double().view(1, H, dk)
            padded = torch.zeros(int(pos[n]) + 1, H, dk, dtype=torch.float64)
            padded[-1] = x[0]
            want = pv.rotate_half_layout(padded, dims, base)[-1] if dims else x[0]
            if which:
                want = want * dk ** -0.5
            # float32 angles at position 1000 are good to 1e-4
            np.testing.assert_allclose(got[n].cpu().view(H, dk).numpy(), want.float().numpy(),
                                       rtol=0, atol=3e-4 * float(x.abs().max()))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_convolution_unit_norms_gates_and_its_state(dtype):
    """The token-parallel half of the delta rule over three calls (5 tokens, 1 token, 1 token:
    the last two read the convolution's inputs from the state only)."""
    from distengine_b200.kernels import recurrent as rk
    H, G, dk, dv, K, T = 3, 1, 10, 6, 4, 7
    g = _gen(1)
    C = 2 * G * dk + H * dv
    b_col = (C + 7) // 8 * 8
    proj = torch.randn(T, b_col + H, generator=g).to(dtype)
    a = torch.randn(T, H * dk, generator=g)
    taps = torch.randn(C, K, generator=g)
    dt_bias, a_log = torch.randn(H * dk, generator=g), torch.randn(H, generator=g) * 0.5
    x = proj[:, :C].double()
    y = pv.silu(pv.causal_conv(x, taps.double()))
    want_q = pv.unit(y[:, : G * dk].view(T, G, dk)) * dk ** -0.5
    want_k = pv.unit(y[:, G * dk: 2 * G * dk].view(T, G, dk))
    want_v = y[:, 2 * G * dk:]
    want_beta = torch.sigmoid(proj[:, b_col:].double())
    want_g = torch.exp(-torch.exp(a_log.double())[None, :, None]
                       * pv.softplus(a.double() + dt_bias.double()).view(T, H, dk))
    rows = H * dk * dv
    state = torch.zeros(3, rows + (K - 1) * C, device=DEV)
    at = 0
    for piece in (5, 1, 1):
        ctx = _ctx((piece,), (at,), (2,))
        bufs = [torch.empty(piece, w, device=DEV) for w in (G * dk, G * dk, H * dv, H, H * dk)]
        p = proj[at: at + piece].to(DEV)
        rk.delta_prep(p, a[at: at + piece].to(DEV).contiguous(), taps.to(DEV), dt_bias.to(DEV),
                      a_log.to(DEV), state, rows, ctx, *bufs, H, G, dk, dv, b_col)
        rk.conv_state(p, state, rows, C, K, ctx)
        sl = slice(at, at + piece)
        tol = torch.float32 if dtype == torch.float32 else torch.bfloat16
        assert_close(bufs[0].view(piece, G, dk), want_q[sl], torch.float32, "q")
        assert_close(bufs[1].view(piece, G, dk), want_k[sl], torch.float32, "k")
        assert_close(bufs[2], want_v[sl], torch.float32, "v")
        assert_close(bufs[3], want_beta[sl], torch.float32, "beta")
        assert_close(bufs[4].view(piece, H, dk), want_g[sl], torch.float32, "decay")
        at += piece
    assert bool((state[:, :rows] == 0).all()) and bool((state[:2] == 0).all())
    assert_close(state[2, rows:].view(K - 1, C), x[T - (K - 1):], torch.float32, "kept inputs")


def _paged(keys, values, page, dtype, seed):
    """keys [T, G, dk], values [T, G, dv] of one sequence in scrambled pages; free pages NaN."""
    T, G, dk = keys.shape
    dv = values.shape[-1]
    need = (T + page - 1) // page
    order = torch.randperm(need + 4, generator=_gen(seed)).tolist()
    kp = torch.full((need + 4, G, page, dk), float("nan"))
    vp = torch.full((need + 4, G, page, dv), float("nan"))
    table = torch.full((3, need + 2), -1, dtype=torch.int32)
    for p in range(need):
        lo, hi = p * page, min((p + 1) * page, T)
        table[1, p] = order[p]
        kp[order[p], :, : hi - lo] = keys[lo:hi].transpose(0, 1)
        vp[order[p], :, : hi - lo] = values[lo:hi].transpose(0, 1)
    return kp.to(DEV, dtype), vp.to(DEV, dtype), table.to(DEV)


def _plain_chunk_attention(q, k, v, r1, r2, scale, size, pos_q):
    """q [n, H, dk] at positions pos_q against all keys k [T, G, dk], v [T, G, dv]."""
    H, G = q.shape[1], k.shape[1]
    k, v = k.repeat_interleave(H // G, 1).double(), v.repeat_interleave(H // G, 1).double()
    out = torch.zeros(q.shape[0], H, v.shape[-1], dtype=torch.float64)
    for n, i in enumerate(pos_q):
        js = torch.arange(i // size * size, i + 1)
        s = torch.einsum("hd,jhd->hj", q[n].double(), k[js]) * scale
        s = s - r1[:, None].double() * torch.log1p(r2[:, None].double() * (i - js)[None].double())
        out[n] = torch.einsum("hj,jhd->hd", torch.softmax(s, dim=-1), v[js])
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,dk,dv,size,page", [(4, 2, 32, 16, 24, 16), (3, 3, 20, 40, 7, 8),
                                                  (6, 1, 12, 70, 50, 32), (2, 2, 96, 64, 100, 16),
                                                  (8, 2, 128, 256, 40, 16), (1, 1, 256, 8, 33, 8)])
def test_chunk_attention_sees_its_chunk_and_nothing_else(dtype, H, G, dk, dv, size, page):
    """A prompt portion and single tokens over the pages.  The key just before every chunk's start
    is made to match the queries far better than any other (seeing it would take the whole
    weight); the chunk's first key is made the best of those that may be seen."""
    from distengine_b200.kernels import recurrent as rk
    from distengine_b200.kernels.attention_plan import build_plan
    T = 2 * size + size // 2 + 3
    g = _gen(size)
    q = torch.randn(T, H, dk, generator=g)
    k = torch.randn(T, G, dk, generator=g)
    v = torch.randn(T, G, dv, generator=g)
    direction = torch.randn(dk, generator=g)
    q = q + 2.0 * direction
    for start in range(size, T, size):
        k[start - 1] = 8.0 * direction                  # just outside
        k[start] = 3.0 * direction                      # just inside
    q, k, v = (t.to(dtype).float() for t in (q, k, v))
    r1, r2 = torch.rand(H, generator=g) + 0.3, torch.rand(H, generator=g) + 0.1
    scale = 0.4 / dk ** 0.5
    kp, vp, table = _paged(k, v, page, dtype, size)
    # a portion that starts inside a chunk and crosses two edges, then tokens one by one
    first = size - 2
    for lo, n in [(first, size + 5)] + [(p, 1) for p in range(first + size + 5, T)]:
        ctx = _ctx((n,), (lo,), (1,))
        rows = rk.chunk_rows_per_tile(dtype, dk, dv, n > 1)
        plan = build_plan(ctx.host.seq_qlen, ctx.host.seq_pos0, H // G, G, rows, 0, chunk=0)
        items = torch.from_numpy(plan.items).to(DEV)
        wide = torch.zeros(n, H * dk + 9, dtype=dtype, device=DEV)
        wide[:, : H * dk] = q[lo: lo + n].reshape(n, -1).to(DEV)
        out = torch.empty(n, H * dv, dtype=dtype, device=DEV)
        rk.chunk_attention(wide, out, kp, vp, table, items, r1.to(DEV), r2.to(DEV), H, G, dk, dv,
                           scale, size, ctx, tile_rows=rows)
        assert int(ctx.status.item()) == 0
        want = _plain_chunk_attention(q[lo: lo + n], k, v, r1, r2, scale, size,
                                      list(range(lo, lo + n)))
        assert_close(out.view(n, H, dv), want, dtype, f"chunk attention at {lo}+{n}")
        if n == 1 and rk.chunk_decode_ok(dtype, H, G, dk, dv):      # the single-token kernel
            out.fill_(float("nan"))
            rk.chunk_attention_decode(wide, out, kp, vp, table, r1.to(DEV), r2.to(DEV), H, G, dk,
                                      dv, scale, size, ctx)
            assert int(ctx.status.item()) == 0
            assert_close(out.view(n, H, dv), want, dtype, f"single-token kernel at {lo}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_values_are_cached_normalised(dtype):
    from distengine_b200.kernels import recurrent as rk
    G, dk, dv, page, n = 2, 12, 20, 8, 5
    g = _gen(9)
    proj = torch.randn(n, 16 + G * (dk + dv), generator=g).to(dtype)
    ctx = _ctx((3, 2), (6, 0), (1, 0))                  # the first sequence crosses a page's end
    table = torch.tensor([[4, -1, -1], [2, 0, -1]], dtype=torch.int32, device=DEV)
    kp = torch.zeros(5, G, page, dk, dtype=dtype, device=DEV)
    vp = torch.zeros(5, G, page, dv, dtype=dtype, device=DEV)
    rk.kv_write_normed(proj.to(DEV), 16, G, dk, dv, 1e-6, kp, vp, table, ctx)
    assert int(ctx.status.item()) == 0
    where = [(2, 6), (2, 7), (0, 0), (4, 0), (4, 1)]    # (page, offset) of the five tokens
    for t, (pid, off) in enumerate(where):
        keys = proj[t, 16: 16 + G * dk].float().view(G, dk)
        vals = pv.rms(proj[t, 16 + G * dk:].double().view(G, dv), 1e-6)
        assert_close(kp[pid, :, off], keys, dtype, "cached key")
        assert_close(vp[pid, :, off], vals, dtype, "cached value")
    assert float(kp.float().abs().sum(dim=(1, 3))[1].sum()) == 0.0       # page 1 untouched


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_head_gates_and_mean_of_normed(dtype):
    from distengine_b200.kernels import recurrent as rk
    n, H, dv, width = 6, 3, 20, 56
    g = _gen(4)
    o = torch.randn(n, H * dv, generator=g) * 5
    gate32 = torch.randn(n, H * dv, generator=g)
    weight = torch.rand(dv, generator=g) + 0.5
    out = torch.empty(n, H * dv, dtype=dtype, device=DEV)
    rk.head_gate(o.to(DEV), gate32.to(DEV), weight.to(DEV), out, H, dv, 1e-5)
    want = (pv.rms(o.double().view(n, H, dv), 1e-5) * weight.double()
            * torch.sigmoid(gate32.double()).view(n, H, dv))
    assert_close(out.view(n, H, dv), want, dtype, "sigmoid gate")
    gate = torch.randn(n, H * dv + 8, generator=g).to(dtype)
    rk.head_gate(o.to(DEV), gate.to(DEV)[:, 8:], None, out, H, dv, 1e-5)
    want = pv.rms(o.double().view(n, H, dv), 1e-5) * pv.silu(gate[:, 8:].double()).view(n, H, dv)
    assert_close(out.view(n, H, dv), want, dtype, "silu gate")
    a = (torch.randn(n, width, generator=g) * 4).to(dtype)
    b = (torch.randn(n, width, generator=g) * 0.1).to(dtype)
    wa, wb = torch.rand(width, generator=g) + 0.5, torch.rand(width, generator=g) + 0.5
    mixed = torch.empty(n, width, dtype=dtype, device=DEV)
    rk.mean_of_normed(a.to(DEV), b.to(DEV), wa.to(DEV), wb.to(DEV), mixed, 1e-6)
    want = 0.5 * (pv.rms(a.double(), 1e-6) * wa.double() + pv.rms(b.double(), 1e-6) * wb.double())
    assert_close(mixed, want, dtype, "mean of normed branches")
