"""Each mechanism of the Sebilorn parts alone: its kernels against the plain function in
``plain_sebilorn``, at sizes that are no multiple of anything, with states carried from one call to
the next, and with inputs made so that a key one position outside a window, a lost kept token, a
far token in a state or a missing soft cap would show."""

from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_sebilorn as ps
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


# ----------------------------------------------------------------------------- row-wise kernels
@pytest.mark.parametrize("width", [5, 40, 257, 1024, 4100])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_layer_norm_with_the_residual_sum(width, dtype):
    from distengine_b200.kernels import ops
    g = _gen(width)
    resid = torch.randn(7, width, generator=g) * 3 + 5.0          # a mean far from zero
    delta = torch.randn(7, width, generator=g).to(dtype)
    weight = (torch.rand(width, generator=g) + 0.5).to(dtype)
    bias = torch.randn(width, generator=g).to(dtype)
    want = ps.layer_norm((resid + delta.float()).double(), weight.double(), bias.double(), 1e-5)
    r = resid.to(DEV)
    out = torch.empty(7, width, dtype=dtype, device=DEV)
    ops.add_layernorm(r, delta.to(DEV), weight.to(DEV), bias.to(DEV), 1e-5, out)
    assert_close(out, want, dtype, "layer norm")
    assert_close(r, resid + delta.float(), torch.float32, "residual sum")
    rows = torch.tensor([5, 0, 5], dtype=torch.int32, device=DEV)
    picked = torch.empty(3, width, dtype=dtype, device=DEV)
    ops.add_layernorm(r, None, weight.to(DEV), bias.to(DEV), 1e-5, picked, rows)
    assert_close(picked, want[[5, 0, 5]], dtype, "layer norm of picked rows")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_activations_scaled_sum_soft_cap_and_scaled_embedding(dtype):
    from distengine_b200.kernels import ops
    g = _gen(1)
    x = (torch.randn(9, 50, generator=g) * 2).to(dtype)
    wide = torch.zeros(9, 64, dtype=dtype)
    wide[:, 8:58] = x
    plain = {"relu2": lambda t: torch.relu(t) ** 2, "tanh": torch.tanh, "silu": ps.silu,
             "gelu_tanh": lambda t: torch.nn.functional.gelu(t, approximate="tanh")}
    for kind, fn in plain.items():
        buf = wide.to(DEV)
        view = buf[:, 8:58]                                  # a block of columns, in place
        ops.activation(view, view, kind)
        assert_close(view, fn(x.double()), dtype, kind)
        assert bool((buf[:, :8] == 0).all()) and bool((buf[:, 58:] == 0).all())
    a, b = torch.randn(6, 33, generator=g), torch.randn(6, 33, generator=g)
    out = torch.empty(6, 33, dtype=dtype, device=DEV)
    ops.scaled_sum(a.to(DEV), b.to(DEV), 0.6, -1.5, out)
    assert_close(out, 0.6 * a.double() - 1.5 * b.double(), dtype, "scaled sum")
    logits = (torch.randn(4, 77, generator=g) * 20).to(DEV)
    want = 7.0 * torch.tanh(logits.double().cpu() / 7.0)
    ops.softcap_(logits, 7.0)
    assert_close(logits, want, torch.float32, "soft cap")
    table = torch.randn(11, 24, generator=g).to(dtype)
    ids = torch.tensor([3, 10, 0, 3], dtype=torch.int32, device=DEV)
    rows = torch.empty(4, 24, device=DEV)
    ops.embed_rows(ids, table.to(DEV), rows, 6.5)
    assert_close(rows, table.double()[[3, 10, 0, 3]] * 6.5, torch.float32, "scaled embedding")


# ----------------------------------------------------------------------------- recurrences
def _delta_inputs(T, H, dk, seed):
    g = _gen(seed)
    r = torch.randn(T, H, dk, generator=g)
    k = torch.randn(T, H, dk, generator=g) * 0.7
    v = torch.randn(T, H, dk, generator=g)
    decay = torch.exp(-0.6 * torch.rand(T, H, dk, generator=g))
    rate = torch.rand(T, H, dk, generator=g)
    return r, k, v, decay, rate


@pytest.mark.parametrize("H,dk", [(2, 20), (1, 68), (3, 5), (2, 128), (1, 160)])
def test_generalized_delta_rule_scan_carries_its_state(H, dk):
    """Two sequences in unequal pieces over three calls, in slots 3 and 1 of 5; the state of an
    untouched slot stays as it is.  z is formed as the preparation kernel forms it."""
    from distengine_b200.kernels import recurrent as rk
    lens = (37, 20)
    data = [_delta_inputs(n, H, dk, 10 + i) for i, n in enumerate(lens)]
    want = [ps.generalized_delta_rule(*(t.double() for t in d)) for d in data]
    state = torch.zeros(5, H * dk * dk + 11, device=DEV)
    state[2] = 7.0
    slots, fed = (3, 1), [0, 0]
    got = [torch.zeros(n, H, dk) for n in lens]
    for pieces in ((30, 1), (1, 17), (6, 2)):
        ctx = _ctx(pieces, fed, slots)
        def cut(fn):
            return torch.cat([fn(*(t[fed[s]: fed[s] + pieces[s]] for t in data[s]))
                              .reshape(pieces[s], -1) for s in range(2)]).to(DEV).contiguous()
        zf = lambda r, k, v, w, a: a * k / ((k * k).sum(-1, keepdim=True) + 1e-6)
        z = cut(zf)
        dots = cut(lambda r, k, v, w, a: torch.stack(((zf(r, k, v, w, a) * r).sum(-1),
                                                      (k * r).sum(-1)), dim=-1))
        out = torch.empty(sum(pieces), H * dk, device=DEV)
        rk.state_scan(cut(lambda r, k, v, w, a: r), cut(lambda r, k, v, w, a: k),
                      cut(lambda r, k, v, w, a: v), state, out, H, H, dk, dk, ctx,
                      g=cut(lambda r, k, v, w, a: w), z=z, dots=dots)
        at = 0
        for s in range(2):
            got[s][fed[s]: fed[s] + pieces[s]] = out[at: at + pieces[s]].cpu().view(-1, H, dk)
            at += pieces[s]
            fed[s] += pieces[s]
    for s in range(2):
        assert_close(got[s], want[s], torch.float32, f"generalized delta rule, sequence {s}")
    assert bool((state[2] == 7.0).all()) and bool((state[0] == 0).all())
    assert bool((state[3, H * dk * dk:] == 0).all())


def test_generalized_delta_rule_removes_along_the_unit_key():
    """No decay (w = 1) and removal rate 1: writing the same key twice leaves the second value
    only, up to the 1e-6 under the root, whatever the key's length - which a removal along the raw
    key, or one that reads the decayed state, would not give."""
    from distengine_b200.kernels import recurrent as rk
    H, dk = 1, 8
    k = torch.zeros(3, H, dk)
    k[0, 0, 2] = k[1, 0, 2] = 3.0
    k[2, 0, 5] = 1.0
    v = torch.tensor([[1.0] * dk, [-2.0] * dk, [0.0] * dk]).view(3, H, dk)
    r = torch.zeros(3, H, dk)
    r[:, 0, 2] = 1.0
    ones = torch.ones(3, H, dk)
    want = ps.generalized_delta_rule(r.double(), k.double(), v.double(), ones.double(),
                                     ones.double())
    assert abs(want[1, 0, 0].item() + 6.0) < 1e-4               # 3 * (-2): the first value is gone
    ctx = _ctx((3,), (0,), (0,))
    flat = lambda t: t.reshape(3, -1).to(DEV).contiguous()
    state = torch.zeros(1, H * dk * dk, device=DEV)
    out = torch.empty(3, H * dk, device=DEV)
    z = ones * k / ((k * k).sum(-1, keepdim=True) + 1e-6)
    dots = torch.stack(((z * r).sum(-1), (k * r).sum(-1)), dim=-1)
    rk.state_scan(flat(r), flat(k), flat(v), state, out, H, H, dk, dk, ctx, g=flat(ones),
                  z=flat(z), dots=flat(dots))
    assert_close(out.view(3, H, dk), want, torch.float32, "removal along the unit key")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_generalized_delta_preparation(dtype):
    from distengine_b200.kernels import recurrent as rk
    n, H, dk = 6, 3, 10
    g = _gen(4)
    rows = H * dk
    proj = torch.randn(n, 5 * rows + 7, generator=g).to(dtype)
    wl = torch.randn(n, rows, generator=g) * 2
    w0, a_bias = torch.randn(rows, generator=g), torch.randn(rows, generator=g)
    outs = [torch.empty(n, rows, device=DEV) for _ in range(4)]
    dots = torch.empty(n, 2 * H, device=DEV)
    rk.gdelta_prep(proj.to(DEV), 0, rows, 4 * rows, wl.to(DEV), w0.to(DEV), a_bias.to(DEV),
                   *outs, dots, H, dk)
    p = proj.double()
    k = p[:, rows: 2 * rows].view(n, H, dk)
    a = torch.sigmoid(p[:, 4 * rows: 5 * rows] + a_bias.double()).view(n, H, dk)
    assert_close(outs[0], p[:, :rows], torch.float32, "r")
    assert_close(outs[1], p[:, rows: 2 * rows], torch.float32, "k")
    assert_close(outs[2], torch.exp(-np.exp(-0.5) * torch.sigmoid(wl.double() + w0.double())),
                 torch.float32, "decay")
    # (a u)(u^T S) with the unit key u = k / sqrt(|k|^2 + 1e-6) is z (k^T S)
    z = a * k / ((k * k).sum(-1, keepdim=True) + 1e-6)
    assert_close(outs[3], z.reshape(n, rows), torch.float32, "z")
    r = p[:, :rows].view(n, H, dk)
    assert_close(dots.view(n, H, 2), torch.stack(((z * r).sum(-1), (k * r).sum(-1)), dim=-1),
                 torch.float32, "z . r and k . r")


def test_lightning_state_keeps_a_far_token():
    """No decay (1.0) and a query that points at the first token's key: 300 tokens later the
    read-out holds that token's value; with decay 0.5 it is gone."""
    from distengine_b200.kernels import recurrent as rk
    T, H, dk, dv = 301, 2, 12, 40
    g = _gen(3)
    k = torch.rand(T, H, dk, generator=g) * 0.01
    q = torch.rand(T, H, dk, generator=g) * 0.05
    v = torch.randn(T, H, dv, generator=g)
    k[:, :, 3] = 0                                   # only the first token's key has channel 3
    k[0, :, 3] = 4.0
    q[300] = 0
    q[300, :, 3] = 4.0
    decay = torch.tensor([1.0, 0.5])
    want = ps.decayed_state(q.double(), k.double(), v.double(), decay.double())
    assert (want[300, 0] - 16 * v[0, 0].double()).abs().max() < 1e-6
    assert want[300, 1].abs().max() < 0.1
    state = torch.zeros(2, H * dk * dv, device=DEV)
    got = torch.empty(T, H * dv)
    fed = 0
    for piece in (200, 1, 1, 99):
        ctx = _ctx((piece,), (fed,), (1,))
        cut = lambda t: t[fed: fed + piece].reshape(piece, -1).to(DEV).contiguous()
        out = torch.empty(piece, H * dv, device=DEV)
        rk.state_scan(cut(q), cut(k), cut(v), state, out, H, H, dk, dv, ctx, decay=decay.to(DEV))
        got[fed: fed + piece] = out.cpu()
        fed += piece
    assert_close(got.view(T, H, dv), want, torch.float32, "lightning state")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gate_with_a_weight_that_spans_the_heads(dtype):
    """Per head (the delta rule's read-out) and over the whole row (lightning: heads 1)."""
    from distengine_b200.kernels import recurrent as rk
    n, H, dv = 5, 3, 20
    g = _gen(8)
    o = torch.randn(n, H * dv, generator=g) * 4
    gate = torch.randn(n, H * dv + 9, generator=g).to(dtype)
    weight = torch.rand(H * dv, generator=g) + 0.5
    sig = torch.sigmoid(gate.double()[:, 4: 4 + H * dv])
    for heads, size in ((H, dv), (1, H * dv)):
        out = torch.empty(n, H * dv, dtype=dtype, device=DEV)
        rk.head_gate(o.to(DEV), gate.to(DEV)[:, 4: 4 + H * dv], weight.to(DEV), out, heads, size,
                     1e-5, spanning=True)
        want = ps.rms(o.double().view(n, heads, size), 1e-5).reshape(n, -1) * weight.double() * sig
        assert_close(out, want, dtype, f"gate, {heads} head(s)")


# ----------------------------------------------------------------------------- attention
class _Pages:
    """A paged cache of one layer with a scrambled block table; free pages hold NaN."""

    def __init__(self, lens, G, dk, dv, page, dtype, seed):
        g = _gen(seed)
        need = [(n + page - 1) // page for n in lens]
        total = sum(need) + 4
        order = torch.randperm(total, generator=g).tolist()
        self.slots = torch.randperm(len(lens) + 2, generator=g)[: len(lens)].tolist()
        self.table = torch.full((len(lens) + 2, max(need) + 1), -1, dtype=torch.int32)
        at = 0
        for s, n in enumerate(need):
            for p in range(n):
                self.table[self.slots[s], p] = order[at]
                at += 1
        self.table = self.table.to(DEV)
        self.k = torch.full((total, G, page, dk), float("nan"), dtype=dtype, device=DEV)
        self.v = torch.full((total, G, page, dv), float("nan"), dtype=dtype, device=DEV)


def _attend(q, k, v, pages, pieces_list, H, G, dk, dv, dtype, rot, fk, fv, scale, window, keep,
            softcap, gate=None):
    """Feed the sequences in the given pieces through kv_write_rotated, the attention kernels and
    attention_finish - or, for steps of single tokens at sizes it takes, through the one kernel
    that does all of it; returns one [T, H dv] tensor a sequence."""
    from distengine_b200.kernels import recurrent as rk
    from distengine_b200.kernels.attention_plan import build_plan
    lens = [x.shape[0] for x in q]
    got = [torch.zeros(n, H * dv) for n in lens]
    fed = [0] * len(lens)
    for pieces in pieces_list:
        live = [s for s in range(len(lens)) if pieces[s] > 0]
        ctx = _ctx([pieces[s] for s in live], [fed[s] for s in live],
                   [pages.slots[s] for s in live])
        rows = [torch.cat((q[s][fed[s]: fed[s] + pieces[s]].reshape(pieces[s], -1),
                           k[s][fed[s]: fed[s] + pieces[s]].reshape(pieces[s], -1),
                           v[s][fed[s]: fed[s] + pieces[s]].reshape(pieces[s], -1)), dim=1)
                for s in live]
        proj = torch.cat(rows).to(dtype).to(DEV).contiguous()
        n = proj.shape[0]
        gt = None
        if gate is not None:
            gt = torch.cat([gate[s][fed[s]: fed[s] + pieces[s]] for s in live]).to(dtype).to(DEV)
        out = torch.empty(n, H * dv, dtype=dtype, device=DEV)
        single = max(pieces) == 1 and rk.chunk_decode_ok(dtype, H, G, dk, dv)
        if single:
            # one kernel: rotation, cache write, attention, back-rotation, gate (q stays as it is)
            before = proj.clone()
            rk.chunk_attention_decode(proj, out, pages.k, pages.v, pages.table, None, None, H, G,
                                      dk, dv, scale, 0, ctx, window=window, keep_first=keep,
                                      softcap=softcap,
                                      fused=dict(fk=fk, rotary_dim=rot, fv=fv, write_kv=True,
                                                 gate=gt))
            assert int(ctx.status.item()) == 0 and torch.equal(proj, before)
            at = 0
            for s in live:
                got[s][fed[s]: fed[s] + pieces[s]] = out[at: at + pieces[s]].float().cpu()
                at += pieces[s]
                fed[s] += pieces[s]
            continue
        rk.kv_write_rotated(proj, fk, rot, fv, H, G, dk, dv, pages.k, pages.v, pages.table, True,
                            ctx)
        raw = torch.empty(n, H * dv, device=DEV)
        # (tiles of 64 rows from 48 rows a portion on, whatever the step's number of blocks)
        tile = rk.chunk_rows_per_tile(dtype, dk, dv, max(pieces) > 1, max(pieces) * (H // G))
        plan = build_plan(ctx.host.seq_qlen, ctx.host.seq_pos0, H // G, G, tile, 0, chunk=0)
        items = torch.from_numpy(plan.items).to(DEV)
        rk.chunk_attention(proj, raw, pages.k, pages.v, pages.table, items, None, None, H, G,
                           dk, dv, scale, 0, ctx, tile_rows=tile, window=window,
                           keep_first=keep, softcap=softcap)
        assert int(ctx.status.item()) == 0
        rk.attention_finish(raw, fv, gt, out, H, dv, ctx)
        at = 0
        for s in live:
            got[s][fed[s]: fed[s] + pieces[s]] = out[at: at + pieces[s]].float().cpu()
            at += pieces[s]
            fed[s] += pieces[s]
    return got


def _plain_attention(q, k, v, dtype, fk, fv, scale, window, keep, softcap, gate=None):
    act = None if dtype == torch.float32 else dtype
    T = q.shape[0]
    pos = torch.arange(T)
    qd, kd, vd = (ps.rnd(t.double(), act) for t in (q, k, v))
    qr = ps.rnd(ps.rotate(qd, pos, fk.double().cpu()), act)
    kr = ps.rnd(ps.rotate(kd, pos, fk.double().cpu()), act)
    vr = ps.rnd(ps.rotate(vd, pos, fv.double().cpu()), act) if fv is not None else vd
    o = ps.softmax_attention(qr, kr, vr, scale, ps.visible(T, window or None, keep),
                             softcap or None)
    if fv is not None:
        o = ps.rotate(o, pos, fv.double().cpu(), sign=-1.0)
    o = o.reshape(T, -1)
    if gate is not None:
        o = o * torch.sigmoid(ps.rnd(gate.double(), act))
    return o


# (H, G, dk, dv, page): odd sizes take the general kernel; whole 16-byte rows the one that loads
# them so, from 48 rows a portion on the one that tiles its products in registers and, for single
# tokens, the one that takes a (sequence, kv head) a block
SHAPES = [(4, 2, 10, 6, 8), (8, 1, 32, 64, 16), (3, 3, 24, 16, 4), (16, 1, 16, 8, 16),
          (4, 2, 128, 128, 16), (2, 1, 40, 200, 8)]


@pytest.mark.parametrize("H,G,dk,dv,page", SHAPES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window,keep,softcap", [(0, 0, 0.0), (13, 0, 4.0), (20, 5, 0.0),
                                                 (9, 37, 7.0), (1, 1, 0.0)])
def test_window_attention_in_portions_and_single_tokens(H, G, dk, dv, page, dtype, window, keep,
                                                        softcap):
    from distengine_b200.parts.window_attention import rotary_frequencies
    lens = (75, 41)
    g = _gen(H * 100 + window)
    q = [torch.randn(n, H, dk, generator=g) for n in lens]
    k = [torch.randn(n, G, dk, generator=g) for n in lens]
    v = [torch.randn(n, G, dv, generator=g) for n in lens]
    gate = [torch.randn(n, H * dv, generator=g) for n in lens]
    rot = dk // 4 * 2
    fk = rotary_frequencies(100.0, rot, (4.0, 1.0, 4.0, 32)).to(DEV)
    fv = rotary_frequencies(100.0, dv).to(DEV) if dv % 2 == 0 else None
    pages = _Pages(lens, G, dk, dv, page, dtype, 5)
    # a portion that crosses the window's and the kept tokens' edges, then single tokens of both
    # sequences together, a step that leaves one sequence out, a portion beside a single token
    pieces = [(30, 2), (1, 1)] + [(1, 1)] * 6 + [(1, 0), (25, 1), (2, 17), (10, 14)]
    got = _attend(q, k, v, pages, pieces, H, G, dk, dv, dtype, rot, fk, fv, 0.3, window, keep,
                  softcap, gate)
    for s in range(2):
        want = _plain_attention(q[s], k[s], v[s], dtype, fk, fv, 0.3, window, keep, softcap,
                                gate[s])
        assert_close(got[s], want, dtype, f"attention, sequence {s}")


@pytest.mark.parametrize("H,G,dk,dv,page", SHAPES[:3])
@pytest.mark.parametrize("single", [False, True])
def test_keys_just_inside_and_outside_window_and_kept_tokens(H, G, dk, dv, page, single):
    """One query and key pair is scaled so that its score stands out: the key just outside the
    window must not be seen, the one just inside must take all the weight; the same for the last
    kept first token against the first one that is not kept - far away, across page borders."""
    from distengine_b200.parts.window_attention import rotary_frequencies
    T, window, keep = 150, 21, 6
    fk = rotary_frequencies(10.0, 0).to(DEV)
    for target in ("outside", "inside", "kept", "not kept"):
        g = _gen(7)
        q = torch.randn(T, H, dk, generator=g) * 0.1
        k = torch.randn(T, G, dk, generator=g) * 0.1
        v = torch.randn(T, G, dv, generator=g)
        i = T - 1
        j = {"outside": i - window, "inside": i - window + 1, "kept": keep - 1,
             "not kept": keep}[target]
        q[i] = 0
        q[i, :, 1] = 9.0
        k[j, :, 1] = 9.0
        pages = _Pages((T,), G, dk, dv, page, torch.float32, 2)
        pieces = [(T - 1,), (1,)] if single else [(T - 40,), (40,)]
        got = _attend([q], [k], [v], pages, pieces, H, G, dk, dv, torch.float32, 0, fk, None, 1.0,
                      window, keep, 0.0)[0]
        want = _plain_attention(q, k, v, torch.float32, fk, None, 1.0, window, keep, 0.0)
        assert_close(got, want, torch.float32, f"{target} key")
        row = got[i].view(H, dv)
        hit = (row - v[j].repeat_interleave(H // G, 0)).abs().max().item()
        if target in ("inside", "kept"):
            assert hit < 1e-3, f"the {target} key does not take the weight"
        else:
            assert hit > 1e-2, f"the {target} key is seen"


def test_soft_cap_bounds_a_large_score():
    """Without the cap a score of 40 takes all the weight; capped at 2 it is one among many."""
    from distengine_b200.parts.window_attention import rotary_frequencies
    H, G, dk, dv, T = 2, 1, 8, 8, 40
    g = _gen(9)
    q = torch.randn(T, H, dk, generator=g) * 0.1
    k = torch.randn(T, G, dk, generator=g) * 0.1
    v = torch.randn(T, G, dv, generator=g)
    q[T - 1, :, 0] = 10.0
    k[3, :, 0] = 4.0
    fk = rotary_frequencies(10.0, 0).to(DEV)
    for softcap in (0.0, 2.0):
        pages = _Pages((T,), G, dk, dv, 16, torch.float32, 1)
        got = _attend([q], [k], [v], pages, [(T,)], H, G, dk, dv, torch.float32, 0, fk, None, 1.0,
                      0, 0, softcap)[0]
        want = _plain_attention(q, k, v, torch.float32, fk, None, 1.0, 0, 0, softcap)
        assert_close(got, want, torch.float32, f"soft cap {softcap}")
        hit = (got[T - 1].view(H, dv) - v[3]).abs().max().item()
        assert (hit < 1e-3) == (softcap == 0.0)
