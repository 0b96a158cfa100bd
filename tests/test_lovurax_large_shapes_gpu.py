"""Lovurax at the layer sizes of real models (one layer of each kind, heads of 64 and of 128 numbers, a latent of 256, four query
heads a key/value head, a retention of eight heads of 64 x 128), against the plain implementation: a prompt of 600 tokens in one
step (the tensor-core kernels and the chunked retention in bfloat16, the 32-bit kernels in float32), then a portion beside nothing
and tokens decoded through captured steps."""
import pytest
import torch

from tests import helpers as H
from tests import lovurax_models as LM
from tests.plain import lovurax_plain as P
from tests.test_lovurax import Run, position_errors

pytestmark = pytest.mark.gpu

BIG = LM.config([(LM.retention(heads=8, dim=64, vdim=128, decay=[1.0 - 2.0 ** -(3 + h) for h in range(8)], rot=32, base=10000.0), LM.dense(ff=2048)),
                 (LM.attention(heads=16, kv_heads=4, dim=64, vdim=64, scale=0.125, coef=0.2, every=128), None),
                 (LM.latent(heads=16, dim=64, vdim=64, rank=256, scale=0.125), LM.dense(ff=2048)),
                 (LM.attention(heads=8, kv_heads=2, dim=128, vdim=128, scale=0.09, coef=0.1, every=500), LM.dense(ff=1024))],
                width=1024, vocab=4099, logit_scale=1.3)


@pytest.fixture(scope="module")
def big(tmp_path_factory):
    tensors = LM.draw_tensors(BIG, seed=31, std=0.1)
    folder = LM.write_model(tmp_path_factory.mktemp("lovurax_big"), BIG, tensors)
    ids = H.random_ids(640, BIG["vocab"], seed=32)
    weights = {k: v.cuda() for k, v in LM.plain_weights(tensors).items()}
    want = _plain_on_gpu(weights, ids)
    return folder, ids, want


def _plain_on_gpu(weights, ids):
    """The plain implementation with its tensors on the device (its loops are the same; only the products are quicker)."""
    default = torch.get_default_device()
    torch.set_default_device("cuda")
    try:
        return P.forward(BIG, weights, ids).cpu()
    finally:
        torch.set_default_device(default)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_real_layer_sizes_in_one_step_in_portions_and_decoded(big, dtype):
    folder, ids, want = big
    run = Run(folder, BIG, ("gpu", dtype), page_size=16, num_pages=2 * 41 + 4, slots=2)
    run.step([("whole", ids[:600])])
    run.finish("whole")
    run.step([("cut", ids[:333])])
    run.step([("cut", ids[333:620])])
    for t in ids[620:]:
        run.step([("cut", [t])])
    run.finish("cut")
    for rid, n in (("whole", 600), ("cut", 640)):
        got = torch.cat(run.logits.pop(rid))
        errs = position_errors(got, want[:n])
        rms = H.rms_error(got, want[:n])
        print(f"MEASURED lovurax real sizes {rid} {dtype}: worst position's error {float(errs.max()):.3e}, rms error {rms:.3e}")
        assert float(errs.max()) < (1e-3 if dtype == torch.float32 else 0.15) and rms < (3e-5 if dtype == torch.float32 else 0.04)
    assert run.all_free()
