"""Lovurax models drawn at random (layer order, every size, decays, rotations, temperatures, scales), each run through the step
function in random portions and batches with pages and slots used again, against the plain implementation. float32 holds every
draw to tight bounds: faults of indexing (a page, a slot, a tile's or a chunk's edge, a head's group, a distance) show there. In
bfloat16 the runs are held to the median over a request's positions of the per-position error: what they add is that every drawn
size finds a bfloat16 kernel that serves it (heads the tensor-core kernels serve in steps of prompt portions, every other case on
the 32-bit kernels), with the strides and alignments it brings. ``LOVURAX_DRAWS=first:count`` runs other draws than the test's."""
import os
import random

import pytest
import torch

from tests import helpers as H
from tests import lovurax_models as LM
from tests.plain import lovurax_plain as P
from tests.test_lovurax import Run, position_errors

pytestmark = pytest.mark.gpu


def draw_config(seed: int) -> dict:
    rng = random.Random(seed)
    width = rng.choice([24, 40, 64, 72, 96, 136, 200])
    layers = []
    for _ in range(rng.randint(2, 6)):
        kind = rng.choice(["retention", "attention", "latent"])
        if kind == "retention":
            heads = rng.choice([1, 2, 3, 4, 6])
            dim = rng.choice([4, 8, 16, 32, 48, 64, 100, 130])
            layer = LM.retention(heads=heads, dim=dim, vdim=rng.choice([5, 8, 31, 32, 33, 64, 100]),
                                 decay=[1.0 - 2.0 ** -rng.uniform(2.0, 10.0) for _ in range(heads)],
                                 rot=rng.choice([r for r in (2, 4, 8, 16, 32, 48, 64, 100, 130) if r <= dim and r % 2 == 0]),
                                 base=rng.choice([50.0, 10000.0, 1000000.0]))
        elif kind == "attention":
            kv_heads = rng.choice([1, 2, 3, 4])
            dim = rng.choice([4, 6, 8, 16, 24, 32, 48, 64, 128])
            vdim = dim if rng.random() < 0.5 else rng.choice([3, 8, 16, 40, 80, 128])
            layer = LM.attention(heads=kv_heads * rng.choice([1, 2, 3, 4, 8]), kv_heads=kv_heads, dim=dim, vdim=vdim,
                                 scale=rng.choice([0.5, 1.0, 2.0]) / dim ** 0.5, coef=rng.choice([None, 0.1, 0.3, 1.0]),
                                 every=rng.choice([1, 3, 16, 64, 100, 256]))
        else:
            dim = rng.choice([4, 8, 16, 32, 64])
            layer = LM.latent(heads=rng.choice([1, 2, 4, 5, 8]), dim=dim, vdim=rng.choice([3, 8, 16, 40, 80]),
                              rank=rng.choice([4, 12, 16, 32, 64, 96, 200]), scale=rng.choice([0.5, 1.0, 2.0]) / dim ** 0.5)
        layers.append((layer, None if rng.random() < 0.3 else LM.dense(ff=rng.choice([16, 48, 128, 320]))))
    return LM.config(layers, width=width, vocab=rng.randint(50, 700), eps=rng.choice([1e-5, 1e-6]), logit_scale=rng.choice([0.5, 1.0, 2.0, 3.7]))


def run_draw(tmp_path, seed: int, dtype) -> None:
    cfg = draw_config(seed)
    rng = random.Random(seed * 7 + 1)
    tensors = LM.draw_tensors(cfg, seed)
    folder = LM.write_model(tmp_path, cfg, tensors)
    weights = LM.plain_weights(tensors)
    page = rng.choice([4, 8, 16])
    run = Run(folder, cfg, ("gpu", dtype), page_size=page, num_pages=3 * (-(-700 // page)) + 2, slots=3)
    reqs = {f"q{i}": H.random_ids(rng.choice([1, 2, 7, 40, 131, 300, 650]), cfg["vocab"], seed * 13 + i) for i in range(5)}
    waiting, live = list(reqs), {}
    while waiting or live:
        while waiting and len(live) < 3:
            live[waiting.pop(0)] = 0
        entries = []
        for rid in [r for r in live if rng.random() < 0.8] or [next(iter(live))]:
            left = len(reqs[rid]) - live[rid]
            n = 1 if left <= 5 else min(left - 5, rng.choice([2, 3, 9, 17, 33, 64, 200, 600]))
            entries.append((rid, reqs[rid][live[rid] : live[rid] + n]))
            live[rid] += n
        run.step(entries)
        for rid, _ in entries:
            if live[rid] == len(reqs[rid]):
                run.finish(rid)
                del live[rid]
    for rid, ids in reqs.items():
        got = torch.cat(run.logits.pop(rid)).double()
        want = P.forward(cfg, weights, list(ids))
        errs = position_errors(got, want)
        assert torch.isfinite(got).all(), (seed, rid)
        if dtype == torch.float32:
            # A position that rounding the plain implementation's norms and projections to 32 bits moves twenty times further than the
            # median position (a dot product next to zero decides the direction of a retention head's output there) is
            # ill-conditioned, not faulty; it is held to the looser bound only.
            rounded = position_errors(P.forward(cfg, weights, list(ids), rounding=lambda z: z.float().double()), want)
            keep = rounded < min(1e-5, 20.0 * float(rounded.median()))
            assert int((~keep).sum()) <= max(3, len(ids) // 10), (seed, rid, int((~keep).sum()))
            rms = H.rms_error(got[keep], want[keep]) if bool(keep.any()) else 0.0
            assert float(errs.max()) < 5e-3 and float(errs[keep].max() if bool(keep.any()) else 0.0) < 2e-3 and rms < 5e-5, \
                (seed, rid, float(errs.max()), int(errs.argmax()), rms)
        else:
            # the yardstick: what rounding the plain implementation's norms and projections to 16 bits does to this request
            rounded = position_errors(P.forward(cfg, weights, list(ids), rounding=lambda z: z.to(torch.bfloat16).double()), want)
            assert float(errs.median()) < max(0.08, 2.0 * float(rounded.median())), (seed, rid, float(errs.median()), float(rounded.median()))
    assert run.all_free()
    run.model.rt.kernels.check_device_status()


_given = os.environ.get("LOVURAX_DRAWS")
SEEDS = [1, 2, 3, 5, 8, 13, 21, 34]
if _given:
    _first, _count = map(int, _given.split(":"))
    SEEDS = list(range(_first, _first + _count))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("seed", SEEDS)
def test_random_configurations_in_random_portions_and_batches(tmp_path, seed, dtype):
    run_draw(tmp_path, seed, dtype)
