"""Nomivik models drawn at random (layer order, every size, a pair table or none, a token input or none, a looped range, windows,
caps, constants), each run through the step function in random portions and batches with pages and slots used again, against the
plain implementation. float32 holds every draw to tight bounds: faults of indexing (a page, a slot, a window's, a tile's or a
chunk's edge, a head's group, a block of channels) show there. In bfloat16 the runs are held to the median over a request's
positions of the per-position error: what they add is that every drawn size finds a bfloat16 kernel that serves it (keys and
values of one size on the tensor-core kernels in steps of prompt portions, every other case on the 32-bit kernel), with the strides
and alignments it brings. ``NOMIVIK_DRAWS=first:count`` runs other draws than the test's."""
import os
import random

import pytest
import torch

from tests import helpers as H
from tests import nomivik_models as NM
from tests.plain import nomivik_plain as P
from tests.test_nomivik import Run, position_errors

pytestmark = pytest.mark.gpu


def draw_config(seed: int) -> dict:
    rng = random.Random(seed)
    width = rng.choice([24, 40, 64, 72, 96, 136, 200])
    layers = []
    for _ in range(rng.randint(2, 6)):
        if rng.random() < 0.5:
            kv_heads = rng.choice([1, 2, 3, 4])
            dim = rng.choice([4, 6, 8, 16, 24, 32, 64, 128])
            vdim = dim if rng.random() < 0.5 else rng.choice([3, 8, 16, 40, 80])
            rot = rng.choice([r for r in (2, 4, 6, 8, 16, 32, 64, 128) if r <= dim])
            left = NM.attention(heads=kv_heads * rng.choice([1, 2, 3, 4, 8]), kv_heads=kv_heads, dim=dim, vdim=vdim, rot=rot,
                                base=rng.choice([50.0, 10000.0, 1000000.0]), scale=rng.choice([0.05, 0.125, 0.3]) * (16.0 / dim) ** 0.5 * 4.0,
                                window=rng.choice([1, 2, 5, 16, 31, 64, 65, 100, 150, 1000]), softcap=rng.choice([0.5, 5.0, 15.0, 50.0]))
            right = NM.memory(heads=rng.choice([1, 2, 3, 4, 6]), dim=rng.choice([3, 8, 16, 32, 48, 64, 100, 130]), vdim=rng.choice([5, 8, 31, 32, 33, 64, 100]),
                              gate_cap=rng.choice([1.0, 6.0, 10.0, 30.0]))
            layer = NM.parallel(left, right)
        else:
            blocks = rng.choice([1, 2, 3, 4, 8])
            layer = NM.recurrence(width=blocks * rng.choice([1, 3, 8, 20, 40, 80]), blocks=blocks, conv=rng.randint(1, 6))
        layers.append((layer, None if rng.random() < 0.4 else NM.dense(ff=rng.choice([16, 48, 128, 320]))))
    loop = None
    if rng.random() < 0.6:
        a = rng.randrange(len(layers))
        loop = (a, rng.randint(a + 1, len(layers)), rng.randint(1, 3))
    pairs = None if rng.random() < 0.15 else (rng.choice([1, 11, 521, 4099]), rng.choice([0, 1, 131, 1000003]), rng.choice([1, 5, 31, 999983]))
    return NM.config(layers, width=width, vocab=rng.randint(50, 700), eps=rng.choice([1e-5, 1e-6]), pairs=pairs,
                     side=rng.choice([None, 1, 2, 8, 24, 40]), loop=loop)


def run_draw(tmp_path, seed: int, dtype) -> None:
    cfg = draw_config(seed)
    rng = random.Random(seed * 7 + 1)
    tensors = NM.draw_tensors(cfg, seed)
    folder = NM.write_model(tmp_path, cfg, tensors)
    weights = NM.plain_weights(tensors)
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
            # A position that rounding the plain implementation's norms and projections to 32 bits moves twenty times further
            # than the median position (a dot product next to zero decides the direction of the matrix memory's output there) is
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


_given = os.environ.get("NOMIVIK_DRAWS")
SEEDS = [1, 2, 3, 5, 8, 13, 21, 34, 55, 89]
if _given:
    _first, _count = map(int, _given.split(":"))
    SEEDS = list(range(_first, _first + _count))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("seed", SEEDS)
def test_random_configurations_in_random_portions_and_batches(tmp_path, seed, dtype):
    run_draw(tmp_path, seed, dtype)
