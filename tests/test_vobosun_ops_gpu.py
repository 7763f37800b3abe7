"""Each mechanism of the Vobosun architecture alone: the engine's kernel or part against the
plain function of tests/plain/vobosun_plain.py, in 32-bit and (where rounding allows a sharp
bound) in bfloat16.  Inputs are made so that a fault shows: a far key gets a score that stands
out among hundreds, a row's state is carried over portions of one and two tokens beside a
poisoned neighbour, router scores are pushed below zero by their corrections."""

import math

import pytest
import torch

from plain import vobosun_plain as P

pytestmark = pytest.mark.gpu

DEV = "cuda"


def ops():
    from scratch_llm_b200.kernels import ops as o
    return o


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def bf16_exact(t):
    return t.to(torch.bfloat16).float()


def feed(kv_specs, state_specs, dtype, page, portions, run, n_pages=64, slots=3, other=None):
    """Feed one request ("a") in ``portions`` (lists of token counts) through ``run(batch, view,
    t0, t1)`` with a real cache manager, free pages and unused slots poisoned; ``other``: a
    second request's portion sizes, fed beside it as long as it lasts."""
    from scratch_llm_b200.cache import CacheManager
    from scratch_llm_b200.engine.batch import BatchStager, RowInput, build_batch
    from scratch_llm_b200.parts import CacheView
    cm = CacheManager(kv_specs, state_specs, page, n_pages, slots, dtype=dtype, device=DEV,
                      poison_free_pages=True)
    assert cm.admit("junk") is not None            # slot 0 belongs to somebody else
    for st in cm.states:
        for one in (st if isinstance(st, tuple) else (st,)):
            if one is not None:
                one[0].fill_(float("nan"))
    cm.admit("a")
    if other:
        cm.admit("b")
    stager = BatchStager(torch.device(DEV))
    t0 = 0
    outs = []
    for k, n in enumerate(portions):
        rows = [RowInput("a", [0] * n, [])]
        if other and k < len(other):
            rows.insert(0, RowInput("b", [0] * other[k], []))
        for r in rows:
            assert cm.reserve(r.request_id, len(r.tokens))
        batch = build_batch(cm, stager, rows, 10, 1 << 20)
        pages, group = cm.entry_pages(0)
        view = CacheView(pages=pages, block_table=batch.block_tables[group] if group is not None
                         else None, page_size=page, state=cm.states[0])
        off = len(rows[0].tokens) if len(rows) > 1 else 0
        outs.append(run(batch, view, t0, t0 + n, off))
        for r in rows:
            cm.commit(r.request_id, len(r.tokens))
        t0 += n
    return torch.cat(outs, 0)


# ---------------------------------------------------------------- tanh norm and token shift

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [10, 33, 64])
def test_tanh_norm_with_token_shift_over_portions(dtype, width):
    from scratch_llm_b200.parts import StateSpec
    g = torch.Generator().manual_seed(width)
    T = 41
    x = torch.randn((T, width), generator=g) * 2
    w, b, mu = (torch.randn((width,), generator=g) for _ in range(3))
    alpha = 0.7
    want = P.token_shift(P.dyt(x.double(), w.double(), alpha, b.double()), mu.double()).float()
    xb = torch.randn((30, width), generator=g)      # a neighbour in the same steps
    portions, other = [1, 2, 7, 1, 1, 16, 2, 11], [5, 1, 2, 3]

    def run(batch, view, t0, t1, off):
        resid = torch.cat([xb[:off], x[t0:t1]], 0).to(DEV)
        out = torch.empty(resid.shape, dtype=dtype, device=DEV)
        ops().dyt_norm(resid, alpha, w.to(DEV), b.to(DEV), out, None,
                       (mu.to(DEV), view.state, batch.token_row, batch.row_start, batch.row_slot,
                        True))
        if batch.n_multi:
            ops().dyt_state_update(resid, alpha, w.to(DEV), b.to(DEV), view.state,
                                   batch.row_start, batch.row_slot, batch.n_rows, dtype)
        return out[off:].float().cpu()

    got = feed([None], [StateSpec((width,), torch.float32)], dtype, 16, portions, run, other=other)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    torch.testing.assert_close(got, want, rtol=tol, atol=tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [7, 48])
def test_tanh_norm_on_a_branchs_output_chains_with_the_next_norm(dtype, width):
    g = torch.Generator().manual_seed(1)
    n = 9
    resid = torch.randn((n, width), generator=g)
    delta = (torch.randn((n, width), generator=g) * 3).to(dtype)
    w1, b1, w2, b2 = (torch.randn((width,), generator=g) for _ in range(4))
    new = resid.double() + P.dyt(delta.double(), w1.double(), 1.3, b1.double())
    nxt = P.dyt(new, w2.double(), 0.4, b2.double())
    r = resid.clone().to(DEV)
    out = torch.empty((n, width), dtype=dtype, device=DEV)
    ops().dyt_add(r, delta.to(DEV), 1.3, w1.to(DEV), b1.to(DEV), (0.4, w2.to(DEV), b2.to(DEV)), out)
    torch.testing.assert_close(r.cpu(), new.float(), rtol=1e-5, atol=1e-5)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    torch.testing.assert_close(out.float().cpu(), nxt.float(), rtol=tol, atol=tol)
    r2 = resid.clone().to(DEV)
    ops().dyt_add(r2, delta.to(DEV), 1.3, w1.to(DEV), b1.to(DEV))
    assert torch.equal(r2, r)
    # gathered rows (the model's last norm)
    rows = [4, 0, 8]
    out3 = torch.empty((3, width), dtype=dtype, device=DEV)
    ops().dyt_norm(r, 0.4, w2.to(DEV), b2.to(DEV), out3, i32(rows))
    torch.testing.assert_close(out3.float().cpu(), nxt.float()[rows], rtol=tol, atol=tol)


def test_xielu_with_its_two_numbers():
    g = torch.Generator().manual_seed(2)
    z = torch.randn((6, 37), generator=g) * 3
    p, q = torch.tensor(0.3, dtype=torch.float64), torch.tensor(-0.8, dtype=torch.float64)
    want = P.xielu(z.double(), p, q).float()
    sp = lambda v: math.log1p(math.exp(v))  # noqa: E731
    out = torch.empty((6, 37), device=DEV)
    ops().param_act(z.to(DEV), out, "xielu", sp(0.3), 0.5 + sp(-0.8))
    torch.testing.assert_close(out.cpu(), want, rtol=1e-5, atol=1e-6)
    zb = z.reshape(-1)[:216].reshape(9, 24).to(torch.bfloat16)
    outb = torch.empty((9, 24), dtype=torch.bfloat16, device=DEV)
    ops().param_act(zb.to(DEV), outb, "xielu", sp(0.3), 0.5 + sp(-0.8))
    torch.testing.assert_close(outb.float().cpu(), P.xielu(zb.double(), p, q).float(),
                               rtol=1e-2, atol=1e-2)


# -------------------------------------------------------------------------------- attention

def attention_part(m, width, w, dtype, max_position=4096):
    from scratch_llm_b200.parts import BuildContext
    from scratch_llm_b200.parts.attention import GQAttention
    from scratch_llm_b200.parts.position import Rotary
    mixer = GQAttention(width, m["heads"], m["kv_heads"], m["dim"], m["scale"], None,
                        names={"q": "q", "k": "k", "v": "v", "o": "o"}, value_dim=m["vdim"],
                        bias=True)
    ctx = BuildContext(dtype=dtype, device=torch.device(DEV))
    mixer.load(w, ctx)
    rot = m["rot"]
    pos = Rotary(m["dim"] + m["dim"] % 2, rot["base"], max_position, interleaved=False,
                 rot_dims=rot["dims"], scaling_factor=(rot.get("scaling") or {}).get("factor", 1.0))
    pos.load({}, ctx)
    return mixer, pos


ATTENTION = [  # heads, kv heads, dim, vdim, rot dims, factor, page
    (8, 2, 64, 64, 64, 2.0, 16), (4, 2, 64, 32, 48, 1.0, 16), (6, 2, 16, 24, 8, 2.0, 8),
    (3, 3, 20, 12, 6, 1.0, 16), (2, 1, 128, 128, 32, 8.0, 32)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H, G, D, Dv, rot, factor, page", ATTENTION)
@pytest.mark.parametrize("cut", ["whole", "decode", "portions"])
def test_attention_sees_far_keys_and_page_borders(cut, H, G, D, Dv, rot, factor, page, dtype):
    """Queries near the end are made to look for one key each: far back (the first tokens), at
    a page's last place and the next page's first, and their own neighbour."""
    g = torch.Generator().manual_seed(H * D + rot)
    width, T = 40, 330
    m = {"heads": H, "kv_heads": G, "dim": D, "vdim": Dv, "scale": 1.0 / math.sqrt(D),
         "rot": {"base": 5000.0, "dims": rot, "scaling": {"factor": factor}}}
    w = {"q": bf16_exact(torch.randn((H * D, width), generator=g) * width ** -0.5),
         "v": bf16_exact(torch.randn((G * Dv, width), generator=g) * width ** -0.5),
         "o": bf16_exact(torch.randn((width, H * Dv), generator=g) * (H * Dv) ** -0.5),
         "q.b": bf16_exact(torch.randn((H * D,), generator=g) * 0.2),
         "k.b": bf16_exact(torch.randn((G * D,), generator=g) * 0.2),
         "v.b": bf16_exact(torch.randn((G * Dv,), generator=g) * 0.2)}
    # each kv head's key matrix is its first query head's: a token meets its own copy strongly
    w["k"] = torch.cat([w["q"][(h * (H // G)) * D:(h * (H // G) + 1) * D] for h in range(G)], 0)
    x = bf16_exact(torch.randn((T, width), generator=g))
    pairs = [(T - 1, 1), (T - 2, page - 1), (T - 3, page), (T - 4, 5 * page + 1), (T - 6, T - 7)]
    for i, j in pairs:
        x[i] = x[j] = bf16_exact(torch.randn((width,), generator=g) * 3.0)
    want = P.attention_mixer(x.double(), {k: v.double() for k, v in w.items()}, m).float()
    mixer, pos = attention_part(m, width, w, dtype)
    portions = {"whole": [T], "decode": [T - 8] + [1] * 8,
                "portions": [7, 2, 100, 1, 33, 2, 152, 3, 20, 2, 1, 1, 2, 1, 1, 1, 1]}[cut]
    assert sum(portions) == T

    def run(batch, view, t0, t1, off):
        return mixer.forward(x[t0:t1].to(DEV, dtype), batch, view, True, pos).float().cpu()

    got = feed([mixer.kv_spec()], [None], dtype, page, portions, run)
    if dtype == torch.float32:
        torch.testing.assert_close(got, want, rtol=2e-4, atol=2e-4)
    else:
        err = (got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean().sqrt()
        assert err.max() < 0.05, err.max()
        assert err[[i for i, _ in pairs]].max() < 0.05


def test_rotation_of_a_part_of_the_head_with_biases():
    """The rotate-and-store kernel alone: the first entries of each head turn in the split-half
    pairing with scaled frequencies, the rest pass, biases are added first, values only get
    their bias."""
    from scratch_llm_b200.parts import BuildContext
    from scratch_llm_b200.parts.position import Rotary
    g = torch.Generator().manual_seed(5)
    H, G, hd, rot, page, n = 3, 2, 16, 6, 4, 5
    pos = Rotary(hd, 300.0, 64, interleaved=False, rot_dims=rot, scaling_factor=3.0)
    pos.load({}, BuildContext(dtype=torch.float32, device=torch.device(DEV)))
    assert pos.cos.shape == (64, rot // 2)
    qkv = torch.randn((n, (H + 2 * G) * hd), generator=g)
    bias = torch.randn(((H + 2 * G) * hd,), generator=g)
    positions = [0, 1, 2, 3, 40]
    with_bias = (qkv + bias).double()
    q = P.rotate_half_layout(with_bias[:, :H * hd].view(n, H, hd), torch.tensor(positions), rot,
                             300.0, 3.0)
    k = P.rotate_half_layout(with_bias[:, H * hd:(H + G) * hd].view(n, G, hd),
                             torch.tensor(positions), rot, 300.0, 3.0)
    pages = torch.full((12, 2, G, page, hd), float("nan"), device=DEV)
    table = i32([[7, 2, 9, 1, 0, 3, 4, 5, 6, 8, 10]])
    dev = qkv.clone().to(DEV)
    ops().rope_kv_write(dev, i32(positions), i32([0] * n), pos.cos, pos.sin, pages, table, page,
                        H, G, hd, False, True, bias.to(DEV))
    torch.testing.assert_close(dev[:, :H * hd].cpu(), q.reshape(n, -1).float(), rtol=1e-5, atol=1e-5)
    for t, p in enumerate(positions):
        slot = pages[int(table[0, p // page]), :, :, p % page].cpu()
        torch.testing.assert_close(slot[0], k[t].float(), rtol=1e-5, atol=1e-5)
        torch.testing.assert_close(slot[1], with_bias[t, (H + G) * hd:].view(G, hd).float(),
                                   rtol=1e-5, atol=1e-5)


# ------------------------------------------------------------------- generalized delta rule

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H, D", [(2, 64), (3, 24), (1, 128), (4, 9), (2, 16)])
def test_general_delta_over_portions_and_slots(H, D, dtype):
    from scratch_llm_b200.parts import BuildContext
    from scratch_llm_b200.parts.general_delta import GeneralDelta
    g = torch.Generator().manual_seed(H * 100 + D)
    width, T, rank, eps = 48, 75, 5, 1e-5
    m = {"heads": H, "dim": D}
    w = {n: bf16_exact(torch.randn((H * D, width), generator=g) * width ** -0.5) for n in "rkvga"}
    w.update({"a.b": bf16_exact(torch.randn((H * D,), generator=g) * 0.5),
              "w1": bf16_exact(torch.randn((rank, width), generator=g) * width ** -0.5),
              "w2": bf16_exact(torch.randn((H * D, rank), generator=g) * 0.6),
              "w0": bf16_exact(torch.randn((H * D,), generator=g) - 0.5),
              "norm": bf16_exact(torch.randn((H * D,), generator=g) * 0.2 + 1.0),
              "o": bf16_exact(torch.randn((width, H * D), generator=g) * (H * D) ** -0.5)})
    x = bf16_exact(torch.randn((T, width), generator=g))
    xb = bf16_exact(torch.randn((40, width), generator=g))
    want = P.general_delta_mixer(x.double(), {k: v.double() for k, v in w.items()}, m, eps).float()
    mixer = GeneralDelta(width, H, D, eps)
    mixer.load(w, BuildContext(dtype=dtype, device=torch.device(DEV)))
    assert mixer.rank == rank
    portions, other = [1, 2, 17, 1, 1, 16, 2, 33, 2], [3, 1, 20, 2, 14]

    def run(batch, view, t0, t1, off):
        rows = torch.cat([xb[sum(other[:len(seen)]):][:off], x[t0:t1]], 0) if off else x[t0:t1]
        seen.append(off)
        return mixer.forward(rows.to(DEV, dtype), batch, view, True, None)[off:].float().cpu()

    seen = []
    got = feed([None], [mixer.state_spec()], dtype, 16, portions, run, other=other)
    if dtype == torch.float32:
        torch.testing.assert_close(got, want, rtol=2e-4, atol=2e-4)
    else:
        err = (got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean().sqrt()
        assert err.max() < 0.05, err.max()


def test_read_out_norm_with_a_gain_per_head_and_a_sigmoid_gate():
    g = torch.Generator().manual_seed(3)
    n, H, V, eps = 5, 3, 20, 1e-4
    o = torch.randn((n, H * V), generator=g) * 2
    gate = torch.randn((n, H * V + 7), generator=g)
    gain = torch.randn((H * V,), generator=g)
    want = P.rms_unit(o.double().view(n, H, V), eps).reshape(n, H * V) * gain.double() \
        * torch.sigmoid(gate[:, 7:].double())
    out = torch.empty((n, H * V), device=DEV)
    ops().head_norm_gate(o.to(DEV), gate.to(DEV)[:, 7:], gain.to(DEV), eps, out, H, "sigmoid")
    torch.testing.assert_close(out.cpu(), want.float(), rtol=1e-5, atol=1e-5)


# ------------------------------------------------------------------------ routed experts

ROUTERS = [  # experts, identity, top, groups (count, keep), shared, expert size
    (5, 1, 2, (3, 2), 24, 40), (9, 3, 3, (2, 1), 32, 16), (4, 0, 1, None, None, 33),
    (0, 3, 2, None, 16, 8), (9, 0, 4, (3, 2), None, 64), (70, 2, 6, (8, 3), 8, 8)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts, identity, top, groups, shared, ff", ROUTERS)
def test_routed_experts(experts, identity, top, groups, shared, ff, dtype):
    routed_experts_case(experts, identity, top, groups, shared, ff, dtype, width=40, n=150)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_routed_experts_with_many_tokens_per_expert(dtype):
    """Experts with several hundred tokens each and sizes beyond one tile of the grouped
    products in both directions (rows of an expert, features of either product)."""
    routed_experts_case(3, 1, 2, None, 72, 200, dtype, width=320, n=700)


def routed_experts_case(experts, identity, top, groups, shared, ff, dtype, width, n):
    from scratch_llm_b200.parts import BuildContext
    from scratch_llm_b200.parts.routed import RoutedExperts
    g = torch.Generator().manual_seed(experts * 10 + top)
    total = experts + identity
    w = {"router": bf16_exact(torch.randn((total, width), generator=g) * 2 * width ** -0.5),
         # (negative on the whole: many choice scores are below zero, where a barred output
         # that counted as 0 would win)
         "correction": bf16_exact(torch.randn((total,), generator=g) * 0.2 - 0.3)}
    for e in range(experts):
        w[f"e{e}.gate"] = bf16_exact(torch.randn((ff, width), generator=g) * width ** -0.5)
        w[f"e{e}.up"] = bf16_exact(torch.randn((ff, width), generator=g) * width ** -0.5)
        w[f"e{e}.down"] = bf16_exact(torch.randn((width, ff), generator=g) * ff ** -0.5)
    if shared:
        w["shared.gate"] = bf16_exact(torch.randn((shared, width), generator=g) * width ** -0.5)
        w["shared.up"] = bf16_exact(torch.randn((shared, width), generator=g) * width ** -0.5)
        w["shared.down"] = bf16_exact(torch.randn((width, shared), generator=g) * shared ** -0.5)
    x = bf16_exact(torch.randn((n, width), generator=g))
    mlp = {"router": {"experts": experts, "identity": identity, "top": top},
           "shared": {"ff": shared} if shared else None}
    if groups:
        mlp["router"]["groups"] = {"count": groups[0], "keep": groups[1]}
    wd = {k: v.double() for k, v in w.items()}
    want = P.moe_ff(x.double(), wd, mlp).float()
    part = RoutedExperts(width, ff, experts, top, identity, *(groups or (1, 1)), shared)
    part.load(w, BuildContext(dtype=dtype, device=torch.device(DEV)))
    got = part.forward(x.to(DEV, dtype)).float().cpu()
    # the choice itself, in 32-bit from the same inputs
    chosen, weights = P.route(x.double(), wd, mlp["router"])
    ids, wts = ops().moe_route(
        (x @ w["router"].T).to(DEV), w["correction"].to(DEV), None, experts, *(groups or (1, 1)),
        top)[:2]
    assert ids.cpu().tolist() == chosen
    torch.testing.assert_close(wts.cpu().double(), torch.stack(weights), rtol=1e-4, atol=1e-6)
    # steps of few tokens take the router that does everything in one launch: the same choice,
    # and the same output as the tokens got in the large batch (bit for bit in 32-bit)
    few = slice(40, 40 + max(1, 48 // top))
    ids_few, wts_few = ops().moe_route(
        (x[few] @ w["router"].T).to(DEV), w["correction"].to(DEV), None, experts,
        *(groups or (1, 1)), top)[:2]
    assert ids_few.cpu().tolist() == chosen[few]
    got_few = part.forward(x[few].to(DEV, dtype)).float().cpu()
    if dtype == torch.float32:
        assert torch.equal(got_few, got[few])
    else:
        torch.testing.assert_close(got_few, got[few], rtol=2e-2, atol=2e-2)
    if dtype == torch.float32:
        torch.testing.assert_close(got, want, rtol=2e-4, atol=2e-4)
        # one token alone gets what it got in the batch (no sum depends on the batch)
        alone = part.forward(x[17:18].to(DEV, dtype)).float().cpu()
        assert torch.equal(alone[0], got[17])
    else:
        err = (got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean().sqrt()
        assert err.median() < 0.02 and err.quantile(0.9) < 0.05


def test_dense_feed_forward_with_xielu():
    from scratch_llm_b200.parts import BuildContext
    from scratch_llm_b200.parts.feed_forward import ActMLP
    g = torch.Generator().manual_seed(4)
    width, ff, n = 24, 50, 11
    w = {"up": bf16_exact(torch.randn((ff, width), generator=g) * width ** -0.5),
         "down": bf16_exact(torch.randn((width, ff), generator=g) * ff ** -0.5),
         "act": bf16_exact(torch.tensor([0.7, -0.2]))}
    x = bf16_exact(torch.randn((n, width), generator=g) * 2)
    want = P.dense_ff(x.double(), {k: v.double() for k, v in w.items()}).float()
    part = ActMLP(width, ff)
    part.load(w, BuildContext(dtype=torch.float32, device=torch.device(DEV)))
    torch.testing.assert_close(part.forward(x.to(DEV)).cpu(), want, rtol=1e-4, atol=1e-5)
