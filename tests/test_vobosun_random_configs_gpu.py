"""Vobosun configurations drawn at random with fixed seeds (every size, the order of the layers,
head counts and groups, rotated parts, scaling factors, routers, layers that run another layer's
tensors, page sizes), each through a whole and a mixed trace in both precisions against the plain
implementation, free pages poisoned."""

import random

import pytest
import torch

import trace_util as T
import vobosun_util as U
from plain import vobosun_plain as P
from test_vobosun_model_gpu import compare, make_runner

pytestmark = pytest.mark.gpu


def draw_mlp(rng):
    kind = rng.choice(["none", "dense", "moe", "moe"])
    if kind == "none":
        return None
    if kind == "dense":
        return U.dense(rng.choice([24, 56, 100, 160]))
    groups = rng.choice([None, 2, 3, 4])
    if groups is None:
        experts, identity = rng.randint(0, 9), rng.randint(0, 2)
        if experts + identity == 0:
            experts = 1
        top = rng.randint(1, min(4, experts + identity))
        pair = None
    else:
        per = rng.randint(1, 4)
        total = groups * per
        identity = rng.randint(0, min(2, total))
        experts = total - identity
        keep = rng.randint(1, groups)
        top = rng.randint(1, min(4, keep * per))
        pair = (groups, keep)
    return U.moe(rng.choice([8, 24, 40, 64, 136]), experts, top, identity=identity, groups=pair,
                 shared=rng.choice([None, 16, 48]))


def draw(seed):
    rng = random.Random(1000 + seed)
    width = rng.choice([32, 40, 64, 96, 128, 256])
    layers = []
    for _ in range(rng.randint(2, 5)):
        if layers and rng.random() < 0.2:
            j = rng.randrange(len(layers))
            if layers[j].get("weights_of") is None:
                layers.append(U.again(layers, j))
                continue
        if rng.random() < 0.55:
            kv = rng.choice([1, 2, 3])
            heads = kv * rng.choice([1, 2, 4])
            dim = rng.choice([8, 16, 24, 32, 64, 128])
            vdim = rng.choice([None, None, 8, 16, 48, 64])
            rot = rng.choice([dim, dim, 2 * rng.randint(1, dim // 2)])
            layers.append(U.attention_layer(
                heads, kv, dim, vdim=vdim, rot_dims=rot, base=rng.choice([30.0, 10000.0, 200000.0]),
                factor=rng.choice([None, 1.0, 2.0, 4.0, 8.0]), scale=rng.choice([None, 0.05, 0.3]),
                mlp=draw_mlp(rng)))
        else:
            layers.append(U.delta_layer(rng.randint(1, 4), rng.choice([8, 16, 24, 32, 64, 128]),
                                        mlp=draw_mlp(rng)))
    cfg = U.config(rng.choice([50, 128, 301]), width, layers, eps=rng.choice([1e-5, 1e-6, 3e-4]))
    lengths = [rng.randint(1, 140) for _ in range(5)] + [rng.choice([1, 2])]
    return cfg, lengths, rng.choice([8, 16, 32, 64])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(12))
def test_random_configuration(seed, dtype, tmp_path):
    from scratch_llm_b200.kernels import ops
    cfg, lengths, page = draw(seed)
    tensors = U.random_tensors(cfg, 200 + seed, rank=3 + seed % 5)
    folder = U.write_model(cfg, tensors, tmp_path / "m")
    reqs = T.make_requests(cfg["vocab"], lengths, seed=seed)
    want = {rid: P.forward(cfg, tensors, toks).float() for rid, toks in reqs.items()}
    for steps in (T.whole(reqs), T.mixed(reqs, seed=seed)):
        runner = make_runner(folder, dtype, page, T.peak_tokens(steps, round_to=max(64, page)),
                             max_requests=4, poison_free_pages=True)
        with torch.no_grad():
            got = T.run_in_process(runner, steps)
        ops.check_kernel_errors()
        assert len(got) == sum(lengths)
        compare(got, want, dtype)
