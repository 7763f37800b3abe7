"""Each mechanism of the Nilevik architecture alone: the engine's kernel against the plain
function of tests/plain/nilevik_plain.py, in 32-bit and (where rounding allows a sharp
bound) in bfloat16.  Inputs are made so that a fault shows: a key just inside and just outside
a window gets a score that stands out, a sink is large enough to matter, a row's state is
carried over portions of two tokens."""

import math

import pytest
import torch

from plain import nilevik_plain as P

pytestmark = pytest.mark.gpu

DEV = "cuda"


def ops():
    from scratch_llm_b200.kernels import ops as o
    return o


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


# ------------------------------------------------------------------ embedding and the stream

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [10, 33, 64])
def test_embedding_with_sinusoid(dtype, width):
    g = torch.Generator().manual_seed(0)
    table = torch.randn((50, width), generator=g).to(torch.bfloat16).float()
    ids = torch.randint(0, 50, (7,), generator=g)
    positions = torch.tensor([0, 1, 2, 63, 64, 1000, 4095])
    want = table[ids] + P.sinusoid(positions, width, torch.float64).float()
    inv = torch.tensor([10000.0 ** (-2.0 * i / width) for i in range((width + 1) // 2)],
                       dtype=torch.float64).float().to(DEV)
    out = torch.empty((7, width), dtype=torch.float32, device=DEV)
    cast = torch.empty((7, width), dtype=dtype, device=DEV)
    ops().embed_positional(i32(ids.tolist()), i32(positions.tolist()), table.to(DEV, dtype), out,
                           cast, inv_freq=inv)
    # the angle is 32-bit: at position 4095 its rounding alone is 2e-4
    torch.testing.assert_close(out.cpu(), want, rtol=0, atol=6e-4)
    torch.testing.assert_close(out[:3].cpu(), want[:3], rtol=0, atol=2e-6)
    assert torch.equal(cast.float(), out.to(dtype).float())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_add_normed(dtype):
    g = torch.Generator().manual_seed(1)
    n, d, eps = 5, 70, 1e-3
    resid = torch.randn((n, d), generator=g)
    delta = (torch.randn((n, d), generator=g) * 3).to(dtype)
    gain = torch.randn((d,), generator=g)
    want = resid + P.rms_norm(delta.float(), gain, eps)
    r = resid.clone().to(DEV)
    cast = torch.empty((n, d), dtype=dtype, device=DEV)
    ops().add_normed(r, delta.to(DEV), gain.to(DEV), eps, cast)
    torch.testing.assert_close(r.cpu(), want, rtol=1e-5, atol=1e-5)
    assert torch.equal(cast.float(), r.to(dtype).float())


def test_gated_activation_and_gates():
    g = torch.Generator().manual_seed(2)
    gu = torch.randn((6, 2 * 37), generator=g) * 3
    out = torch.empty((6, 37), device=DEV)
    ops().gated_act(gu.to(DEV), out, "gelu_tanh")
    torch.testing.assert_close(out.cpu(), P.gelu_tanh(gu[:, :37]) * gu[:, 37:], rtol=1e-5, atol=1e-6)
    ops().gated_act(gu.to(DEV), out, "silu")
    torch.testing.assert_close(out.cpu(), P.silu(gu[:, :37]) * gu[:, 37:], rtol=1e-5, atol=1e-6)
    # x *= sigmoid(gate), both column slices of wider buffers
    wide = torch.randn((6, 100), generator=g).to(DEV)
    x = wide[:, 10:40].clone()
    ops().sigmoid_gate(x, wide[:, 60:90])
    torch.testing.assert_close(x.cpu(), (wide[:, 10:40] * torch.sigmoid(wide[:, 60:90])).cpu(),
                               rtol=1e-5, atol=1e-6)


def test_token_side_gather():
    g = torch.Generator().manual_seed(3)
    n, dim, layers, vocab = 9, 5, 3, 20
    a = torch.randn((n, dim), generator=g) * 2
    table = torch.randn((vocab, layers * dim), generator=g)
    ids = torch.randint(0, vocab, (n,), generator=g)
    for layer in range(layers):
        out = torch.empty((n, dim), device=DEV)
        ops().side_gate(a.to(DEV), i32(ids.tolist()), table.to(DEV), layer * dim, out, "gelu_tanh")
        want = P.gelu_tanh(a) * table[ids][:, layer * dim:(layer + 1) * dim]
        torch.testing.assert_close(out.cpu(), want, rtol=1e-5, atol=1e-6)


# ------------------------------------------------------------------------------- attention

def fill_pages(k_rows, v_rows, page_size, n_pages, G, hd, dtype, first_page=3, shuffle_seed=0):
    """Pages for one request whose keys/values are ``k_rows`` / ``v_rows`` [T, G, hd], at page
    ids in a shuffled order; every other place holds NaN."""
    T = k_rows.shape[0]
    pages = torch.full((n_pages, 2, G, page_size, hd), float("nan"), dtype=dtype, device=DEV)
    need = -(-T // page_size)
    order = torch.randperm(n_pages - first_page,
                           generator=torch.Generator().manual_seed(shuffle_seed))[:need] + first_page
    for t in range(T):
        p, off = int(order[t // page_size]), t % page_size
        pages[p, 0, :, off] = k_rows[t].to(DEV, dtype)
        pages[p, 1, :, off] = v_rows[t].to(DEV, dtype)
    return pages, i32([order.tolist()])


def plain_attention(q, k, v, pos0, scale, window, slopes, sinks):
    """q [n, H, hd] at positions pos0.., k/v [T, G, hd] -> [n, H, hd], the equations written out."""
    n, H, hd = q.shape
    G = k.shape[1]
    out = torch.zeros((n, H, hd), dtype=torch.float64)
    for h in range(H):
        g = h // (H // G)
        for a in range(n):
            i = pos0 + a
            lo = max(0, i - window + 1) if window else 0
            s = (k[lo:i + 1, g].double() @ q[a, h].double()) * scale
            if slopes is not None:
                s = s - slopes[h] * (i - torch.arange(lo, i + 1)).double()
            e = torch.exp(s - s.max())
            den = e.sum() + (math.exp(sinks[h] - float(s.max())) if sinks is not None else 0.0)
            out[a, h] = (e / den) @ v[lo:i + 1, g].double()
    return out


def run_attention(kind, q, pages, table, page_size, pos0, H, G, hd, scale, window, slopes, sinks,
                  n_splits=1, gate=None, merge_inside=False):
    o = ops()
    n = q.shape[0]
    dtype = pages.dtype
    qd = q.reshape(n, H * hd).to(DEV, dtype).contiguous()
    out = torch.empty_like(qd)
    row_start, row_pos0 = i32([0, n]), i32([pos0])
    sl = None if slopes is None else torch.tensor(slopes, dtype=torch.float32, device=DEV)
    sk = None if sinks is None else torch.tensor(sinks, dtype=torch.float32, device=DEV)
    if kind == "simt":
        o.attention_simt(qd, pages, table, page_size, row_start, row_pos0, out, 1, n, H, G, hd,
                         scale, window, sl, sk)
    elif kind == "tc":
        assert gate is None
        o.attention_tc(qd, pages, table, page_size, row_start, row_pos0, out, i32([0]), 1, n, H, G,
                       hd, scale, window, sl, sk, biased=True)
        assert o.attention_tc_error(hd) == 0
    else:
        scratch = None
        if n_splits > 1:
            scratch = torch.empty(o.attention_mma_scratch_floats(n, H, hd, n_splits),
                                  dtype=torch.float32, device=DEV)
        o.attention_mma(qd, pages, table, page_size, row_start, row_pos0, out, i32([0]), 1, n, H,
                        G, hd, scale, window, split=(kind == "split"), n_splits=n_splits,
                        scratch=scratch, slopes=sl, sinks=sk,
                        gate=None if gate is None else gate.reshape(n, H * hd).to(DEV, dtype),
                        merge_inside=merge_inside)
    return out.float().cpu().view(n, H, hd)


CASES = [  # kind, dtype, head size, new tokens, splits
    ("simt", torch.float32, 16, 40, 1), ("simt", torch.float32, 24, 1, 1),
    ("simt", torch.bfloat16, 40, 7, 1),
    ("wide", torch.bfloat16, 64, 40, 1), ("wide", torch.bfloat16, 32, 90, 1),
    ("split", torch.bfloat16, 64, 1, 1), ("split", torch.bfloat16, 64, 1, 3),
    ("split", torch.bfloat16, 32, 1, 1), ("split", torch.bfloat16, 32, 1, 2),
    # tcgen05: one query tile of 64 tokens x 2 heads, two of them, a ragged second one
    ("tc", torch.bfloat16, 64, 64, 1), ("tc", torch.bfloat16, 64, 100, 1),
    ("tc", torch.bfloat16, 128, 128, 1),
]


@pytest.mark.parametrize("kind, dtype, hd, n_new, n_splits", CASES)
@pytest.mark.parametrize("window", [None, 37, 64])
def test_attention_with_slopes_sink_and_window(kind, dtype, hd, n_new, n_splits, window):
    H, G, page_size, T = 4, 2, 16, 150
    g = torch.Generator().manual_seed(hd + n_new)
    k = torch.randn((T, G, hd), generator=g).to(dtype).float()
    v = torch.randn((T, G, hd), generator=g).to(dtype).float()
    pos0 = T - n_new
    q = torch.randn((n_new, H, hd), generator=g).to(dtype).float()
    slopes = [2.0 ** (-8.0 * (h + 1) / H) for h in range(H)]
    sinks = [1.5, -0.5, 4.0, 0.0]      # one of them above most scores
    pages, table = fill_pages(k, v, page_size, 16, G, hd, dtype)
    scale = 0.4 / math.sqrt(hd)
    got = run_attention(kind, q, pages, table, page_size, pos0, H, G, hd, scale, window, slopes,
                        sinks, n_splits)
    want = plain_attention(q, k, v, pos0, scale, window, slopes, sinks).float()
    tol = dict(rtol=1e-4, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(got, want, **tol)
    # without the sink the result differs: the test would notice a sink that is left out
    no_sink = plain_attention(q, k, v, pos0, scale, window, slopes, None).float()
    assert (no_sink - want).abs().max() > 0.05
    if kind not in ("simt", "tc"):
        # the output gate in the kernel's epilogue, and the splits merged by the last CTA
        gate = torch.randn((n_new, H, hd), generator=g).to(dtype).float() * 2
        for inside in (False, True):
            got = run_attention(kind, q, pages, table, page_size, pos0, H, G, hd, scale, window,
                                slopes, sinks, n_splits, gate=gate, merge_inside=inside)
            torch.testing.assert_close(got, want * torch.sigmoid(gate), **tol)


@pytest.mark.parametrize("kind, dtype, hd, n_new, n_splits", CASES)
def test_a_key_at_the_windows_edge_stands_out(kind, dtype, hd, n_new, n_splits):
    """One key has a huge score with the last query.  Placed at distance window - 1 it takes all
    the weight; at distance window it must not be seen at all."""
    H, G, page_size, window = 2, 1, 16, 50
    T = max(120, n_new + 30)
    g = torch.Generator().manual_seed(7)
    last = T - 1
    for distance, seen in ((window - 1, True), (window, False)):
        k = torch.randn((T, G, hd), generator=g).to(dtype).float() * 0.1
        v = torch.randn((T, G, hd), generator=g).to(dtype).float()
        q = torch.randn((n_new, H, hd), generator=g).to(dtype).float() * 0.1
        j = last - distance
        k[j] = 0.0
        k[j, :, 0] = 8.0
        q[-1, :, 0] = 8.0                       # score 64 * scale with key j, tiny with the rest
        v[j] = 0.0
        v[j, :, 1] = 100.0
        pages, table = fill_pages(k, v, page_size, 16, G, hd, dtype, shuffle_seed=distance)
        got = run_attention(kind, q, pages, table, page_size, T - n_new, H, G, hd, 1.0, window,
                            [0.01, 0.02], [0.0, 0.0], n_splits)
        if seen:
            assert (got[-1, :, 1] > 90).all(), got[-1, :, :3]
        else:
            assert (got[-1, :, 1].abs() < 5).all(), got[-1, :, :3]
        assert torch.isfinite(got).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hd, extra", [(20, 7), (32, 8), (64, 16), (128, 0)])
def test_qk_norm_temperature_and_cache_write(dtype, hd, extra):
    """``extra``: columns behind the heads that the kernel must leave alone (head sizes 8 * 2^k
    with rows of whole 16 bytes take the kernel with 16-byte accesses in bfloat16)."""
    H, G, page_size, eps = 3, 3, 8, 1e-4
    g = torch.Generator().manual_seed(5)
    n = 12
    positions = [0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11]
    x = torch.randn((n, (H + G) * hd + extra), generator=g).to(dtype)
    q_gain, k_gain = torch.randn((hd,), generator=g), torch.randn((hd,), generator=g)
    coef, every = 0.7, 4
    pages = torch.full((4, 2, G, page_size, hd), float("nan"), dtype=dtype, device=DEV)
    table = i32([[2, 0]])
    xd = x.clone().to(DEV)
    ops().qk_norm_kv_write(xd, i32(positions), i32([0] * n), q_gain.to(DEV), k_gain.to(DEV), eps,
                           coef, float(every), None, pages, table, page_size, H, G, hd, True)
    xf = x.float()
    q = xf[:, :H * hd].view(n, H, hd)
    k = xf[:, H * hd:(H + G) * hd].view(n, G, hd)
    temp = torch.tensor([P.query_temperature(p, coef, every) for p in positions]).view(n, 1, 1)
    assert len({round(float(t), 6) for t in temp.flatten()}) >= 3   # the factor does change
    tol = dict(rtol=1e-5, atol=1e-6) if dtype == torch.float32 else dict(rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(xd[:, :H * hd].float().cpu().view(n, H, hd),
                               P.rms_norm(q, q_gain, eps) * temp, **tol)
    assert torch.equal(xd[:, H * hd:].cpu(), x[:, H * hd:])       # keys and the rest untouched
    for t, p in enumerate(positions):
        page, off = [2, 0][p // page_size], p % page_size
        torch.testing.assert_close(pages[page, 0, :, off].float().cpu(),
                                   P.rms_norm(k[t], k_gain, eps), **tol)
        assert torch.equal(pages[page, 1, :, off].float().cpu(), k[t])   # values: keys as projected


# ------------------------------------------------------------------------- recurrent mixer

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("taps", [1, 2, 4])
@pytest.mark.parametrize("C, extra", [(13, 5), (16, 8)])
def test_convolution_carries_its_inputs_over_portions(dtype, taps, C, extra):
    """(16 channels in rows of 24: the bfloat16 kernel with 16-byte accesses and transposed taps)"""
    g = torch.Generator().manual_seed(taps)
    T = 23
    x = torch.randn((T, C + extra), generator=g).to(dtype)
    w = torch.randn((C, taps), generator=g)
    want = P.silu(P.causal_conv(x[:, :C].float(), w))
    state = None if taps == 1 else torch.zeros((3, taps - 1, C), dtype=dtype, device=DEV)
    if state is not None:
        state[0].fill_(float("nan"))            # another request's slot: never read
    got, t = [], 0
    for size in (2, 1, 5, 2, 1, 1, 9, 2):       # portions shorter and longer than the taps
        part = x[t:t + size].to(DEV)
        out = torch.empty((size, C), dtype=dtype, device=DEV)
        row_start, slot, rows = i32([0, size]), i32([2]), i32([0] * size)
        ops().conv_silu(part, w.to(DEV), state, rows, row_start, slot, out,
                        taps_t=w.t().contiguous().to(DEV))
        if taps > 1:
            ops().conv_state_update(part, taps, state, row_start, slot, 1)
        got.append(out.float().cpu())
        t += size
    assert t == T
    tol = dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(torch.cat(got), want, **tol)


def plain_delta(q, k, v, a, b, A_log, dt_bias):
    """[T, G, D], [T, G, D], [T, H, V], gates [T, H] -> read-outs [T, H, V], in 64-bit."""
    T, H, V = v.shape
    G, D = k.shape[1], k.shape[2]
    qn = P.unit_vector(q.double()) * D ** -0.5
    kn = P.unit_vector(k.double())
    beta = torch.sigmoid(b.double())
    decay = torch.exp(-torch.exp(A_log.double()) * torch.nn.functional.softplus(a.double() + dt_bias.double()))
    out = torch.zeros((T, H, V), dtype=torch.float64)
    for h in range(H):
        gk = h // (H // G)
        S = torch.zeros((D, V), dtype=torch.float64)
        for t in range(T):
            S = decay[t, h] * S
            u = beta[t, h] * (v[t, h].double() - S.T @ kn[t, gk])
            S = S + torch.outer(kn[t, gk], u)
            out[t, h] = S.T @ qn[t, gk]
    return out


@pytest.mark.parametrize("H, G, D, V", [(2, 1, 64, 64), (4, 2, 16, 24), (3, 3, 8, 40),
                                        (1, 1, 33, 7), (2, 2, 160, 48)])
def test_delta_rule_over_portions_and_slots(H, G, D, V):
    g = torch.Generator().manual_seed(D)
    T = 70
    q, k = torch.randn((T, G, D), generator=g), torch.randn((T, G, D), generator=g)
    v = torch.randn((T, H, V), generator=g)
    a, b = torch.randn((T, H), generator=g) * 2, torch.randn((T, H), generator=g) * 2
    A_log, dt_bias = torch.randn((H,), generator=g) * 0.5 - 1.0, torch.randn((H,), generator=g)
    want = plain_delta(q, k, v, a, b, A_log, dt_bias).float()
    act = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], 1).to(DEV)
    ab = torch.cat([a, b], 1).to(DEV)
    state = torch.zeros((3, H, V, D), device=DEV)
    state[1].fill_(float("nan"))                # a slot of nobody: never read, never written
    got, t = [], 0
    for size in (17, 1, 2, 16, 1, 1, 32):       # portions around the kernel's chunk of 16 tokens
        out = torch.empty((size, H * V), device=DEV)
        # the portion is row 1 of a batch whose row 0 has no tokens (its slot stays as it is)
        ops().delta_rule(act[t:t + size], ab[t:t + size], A_log.to(DEV), dt_bias.to(DEV), state,
                         i32([0, 0, size]), i32([1, 2]), out, 2, H, G, D, V,
                         max_new=1 if size == 1 and t > 40 else 0)   # (both kernels meet one token)
        got.append(out.cpu().view(size, H, V))
        t += size
    assert t == T
    torch.testing.assert_close(torch.cat(got), want, rtol=2e-4, atol=2e-5)
    assert torch.isnan(state[1]).all() and (state[0] == 0).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_read_out_norm_and_gate(dtype):
    g = torch.Generator().manual_seed(9)
    n, H, V, eps = 6, 3, 20, 1e-5
    o = torch.randn((n, H * V), generator=g) * 4
    wide = torch.randn((n, 10 + H * V), generator=g).to(dtype)
    gain = torch.randn((V,), generator=g)
    out = torch.empty((n, H * V), dtype=dtype, device=DEV)
    ops().head_norm_gate(o.to(DEV), wide.to(DEV)[:, 10:], gain.to(DEV), eps, out, H)
    want = (P.rms_norm(o.view(n, H, V), gain, eps) * P.silu(wide[:, 10:].float()).view(n, H, V))
    tol = dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(out.float().cpu().view(n, H, V), want, **tol)


# ---------------------------------------------------- gate/up products with gelu on the gate

@pytest.mark.parametrize("kernel, m, f, k", [("gemv_mma", 4, 72, 64), ("gemv_mma", 33, 40, 128),
                                            ("gemv_tma", 1, 1536, 1024), ("gemv_tma", 8, 512, 2048),
                                            ("gemm_tc", 300, 200, 256), ("gemm_tc", 1100, 512, 1024)])
def test_fused_gate_up_products_take_the_gelu(kernel, m, f, k):
    """act(x Wg^T) * (x Wu^T) inside the product kernels, against the unfused arithmetic (gate
    and up rounded to bfloat16 first, the activation in 32-bit)."""
    g = torch.Generator().manual_seed(m + f)
    x = (torch.randn((m, k), generator=g)).to(torch.bfloat16)
    w = (torch.randn((2 * f, k), generator=g) * k ** -0.5 * 2).to(torch.bfloat16)
    gu = (x.float() @ w.float().T).to(torch.bfloat16).float()
    out = torch.empty((m, f), dtype=torch.bfloat16, device=DEV)
    o = ops()
    if kernel == "gemv_tma" and not o.gemv_tma_supports(m, 2 * f, k, True):
        pytest.skip("the persistent product does not take this shape on this device")
    for activation, act in (("gelu_tanh", P.gelu_tanh), ("silu", P.silu)):
        getattr(o, kernel)(x.to(DEV), w.to(DEV), out, swiglu=True, activation=activation)
        want = act(gu[:, :f]) * gu[:, f:]
        torch.testing.assert_close(out.float().cpu(), want, rtol=2e-2, atol=2e-2)
    o.check_kernel_errors()
