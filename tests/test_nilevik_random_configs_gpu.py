"""Nilevik configurations drawn at random with fixed seeds (every size, the order of the layers,
windows, periods, taps, page sizes), each through a whole and a mixed trace in both precisions
against the plain implementation, free pages poisoned."""

import random

import pytest
import torch

import nilevik_util as U
import trace_util as T
from plain import nilevik_plain as P
from test_nilevik_model_gpu import compare, make_runner

pytestmark = pytest.mark.gpu


def draw(seed):
    rng = random.Random(seed)
    width = rng.choice([32, 40, 64, 96, 128])
    layers = []
    for _ in range(rng.randint(2, 5)):
        ff = rng.choice([None, rng.choice([24, 56, 100, 160])])
        if rng.random() < 0.55:
            kv = rng.choice([1, 2, 3])
            heads = kv * rng.choice([1, 2, 4])
            dim = rng.choice([16, 32, 48, 64, 128])
            layers.append(U.attention_layer(
                heads, kv, dim, window=rng.choice([1, 5, 16, 23, 64, 100, 1000]),
                scale=rng.choice([None, 0.05, 0.3]), coef=rng.choice([None, 0.2, 1.0]),
                every=rng.choice([1, 4, 9, 128]), ff=ff))
        else:
            kv = rng.choice([1, 2])
            heads = kv * rng.choice([1, 2, 3])
            layers.append(U.delta_layer(heads, kv, rng.choice([8, 16, 32, 64, 128]),
                                        rng.choice([8, 16, 24, 64, 128]),
                                        conv=rng.choice([1, 2, 3, 4]), ff=ff))
    cfg = U.config(rng.choice([50, 128, 301]), width, layers,
                   side_dim=rng.choice([None, 4, 16, 24]), eps=rng.choice([1e-5, 1e-6, 3e-4]))
    lengths = [rng.randint(1, 140) for _ in range(5)] + [rng.choice([1, 2])]
    return cfg, lengths, rng.choice([8, 16, 32, 64])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(10))
def test_random_configuration(seed, dtype, tmp_path):
    cfg, lengths, page = draw(seed)
    tensors = U.random_tensors(cfg, 100 + seed)
    folder = U.write_model(cfg, tensors, tmp_path / "m")
    reqs = T.make_requests(cfg["vocab"], lengths, seed=seed)
    want = {rid: P.forward(cfg, tensors, toks).float() for rid, toks in reqs.items()}
    for steps in (T.whole(reqs), T.mixed(reqs, seed=seed)):
        runner = make_runner(folder, dtype, page, T.peak_tokens(steps, round_to=max(64, page)),
                             max_requests=4, poison_free_pages=True)
        with torch.no_grad():
            got = T.run_in_process(runner, steps)
        assert len(got) == sum(lengths)
        compare(got, want, dtype)
