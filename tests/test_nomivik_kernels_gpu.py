"""The recurrence kernels of the Nomivik parts on the device against the plain formulas of tests/plain/nomivik_plain.py: the gated
linear recurrence and the matrix memory, each walked a row at a time and cut into chunks that run side by side, over rows of
unequal length (none, one token, a chunk exactly, a chunk and one, many chunks), from states that an earlier call left."""
import pytest
import torch

from tests import helpers as H
from tests.plain import nomivik_plain as P

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]
ROWS = [0, 1, 64, 65, 200, 3, 128]          # tokens of every row of a step; the slots are taken in another order


def i32(values):
    return torch.tensor(values, dtype=torch.int32).cuda()


def close(got, want, dtype, what, f32=3e-5, bf16=2e-2):
    err = H.scaled_error(got.float(), want)
    print(f"MEASURED {what} {dtype}: {err:.3e}")
    assert err < (f32 if dtype == torch.float32 else bf16), (what, err)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width,blocks", [(48, 4), (130, 2), (256, 1)])
@pytest.mark.parametrize("chunked", [False, True])
def test_the_gated_recurrence_walked_and_in_chunks(kernels, dtype, width, blocks, chunked):
    g = torch.Generator().manual_seed(width + blocks)
    bw, T = width // blocks, sum(ROWS)
    r = lambda *shape: torch.randn(*shape, generator=g)
    slots = [5, 0, 3, 1, 6, 2, 4]
    indptr = [0]
    for n in ROWS:
        indptr.append(indptr[-1] + n)
    lam, bias = -7.0 + 6.0 * torch.rand(width, generator=g), 0.5 * r(blocks, 2 * bw)
    decay = (8.0 * torch.nn.functional.softplus(lam)).contiguous()
    state = torch.zeros(8, width + 5).cuda()                       # a slot wider than the state: the stride is the slot's
    want_state = torch.zeros(8, width, dtype=torch.float64)
    for call in range(2):                                          # the second call starts from what the first one left
        u, yx = r(T, width).to(dtype), r(T, 2 * width).to(dtype)
        gates = 2.0 * r(blocks, T, 2 * bw)
        out = kernels.gated_recurrence_scan(u.cuda(), gates.cuda(), yx.cuda(), bias.cuda(), decay.cuda(), state, i32(indptr), i32(slots), width, blocks,
                                            chunked=chunked)
        arg = gates.double() + bias.double()[:, None, :]
        rr = P.sigmoid(arg[:, :, :bw]).permute(1, 0, 2).reshape(T, width)
        ii = P.sigmoid(arg[:, :, bw:]).permute(1, 0, 2).reshape(T, width)
        a = torch.exp(-decay.double() * rr)
        drive = torch.sqrt(1.0 - a * a) * ii * u.double()
        want = torch.zeros(T, width, dtype=torch.float64)
        for row, slot in enumerate(slots):
            S = want_state[slot]
            for t in range(indptr[row], indptr[row + 1]):
                S = a[t] * S + drive[t]
                want[t] = S * P.gelu_tanh(yx[t, :width].double())
            want_state[slot] = S
        close(out.cpu(), want, dtype, f"gated recurrence, call {call}")
        close(state[:, :width].cpu(), want_state, torch.float32, f"its state, call {call}")
    assert float(state[:, width:].abs().max()) == 0.0               # nothing written beside the state
    assert float(state[7].abs().max()) == 0.0                       # nor into a slot no row names


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,dim,vdim", [(2, 20, 36), (1, 64, 70), (3, 100, 32), (1, 160, 40), (1, 520, 33)])
@pytest.mark.parametrize("chunked", [False, True])
def test_the_matrix_memory_walked_and_in_chunks(kernels, dtype, heads, dim, vdim, chunked):
    g = torch.Generator().manual_seed(heads * dim + vdim)
    T, cap, floor = sum(ROWS), 6.0, 1e-6
    r = lambda *shape: torch.randn(*shape, generator=g)
    slots = [5, 0, 3, 1, 6, 2, 4]
    indptr = [0]
    for n in ROWS:
        indptr.append(indptr[-1] + n)
    per_head = dim * vdim + dim + 1
    state = torch.zeros(8, heads * per_head + 3).cuda()
    S = torch.zeros(8, heads, dim, vdim, dtype=torch.float64)
    N = torch.zeros(8, heads, dim, dtype=torch.float64)
    M = torch.zeros(8, heads, dtype=torch.float64)
    for call in range(2):
        qkvg = r(T, 2 * heads * dim + 2 * heads * vdim).to(dtype)     # the output gate's columns follow and are not read
        gates = torch.cat([3.0 * r(T, heads), 2.0 + 2.0 * r(T, heads)], dim=1)
        out = kernels.matrix_memory_scan(qkvg.cuda(), gates.cuda(), state, i32(indptr), i32(slots), heads, dim, vdim, cap, floor, chunked=chunked)
        x = qkvg.double()
        q = x[:, : heads * dim].reshape(T, heads, dim) * dim ** -0.5
        k = x[:, heads * dim : 2 * heads * dim].reshape(T, heads, dim)
        v = x[:, 2 * heads * dim : 2 * heads * dim + heads * vdim].reshape(T, heads, vdim)
        gi = cap * torch.tanh(gates[:, :heads].double() / cap)
        gf = P.log_sigmoid(cap * torch.tanh(gates[:, heads:].double() / cap))
        want = torch.zeros(T, heads, vdim, dtype=torch.float64)
        for row, slot in enumerate(slots):
            for t in range(indptr[row], indptr[row + 1]):
                new = torch.maximum(gf[t] + M[slot], gi[t])
                keep, take = torch.exp(gf[t] + M[slot] - new), torch.exp(gi[t] - new)
                S[slot] = keep[:, None, None] * S[slot] + take[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
                N[slot] = keep[:, None] * N[slot] + take[:, None] * k[t]
                M[slot] = new
                den = torch.maximum((N[slot] * q[t]).sum(-1).abs(), torch.exp(-new)) + floor
                want[t] = torch.einsum("hdv,hd->hv", S[slot], q[t]) / den[:, None]
        # an output is a quotient whose denominator can lie next to zero: compared as the kernel's users see it, a head at a time
        # divided by its root mean square
        unit = lambda o: o / torch.sqrt((o * o).mean(-1, keepdim=True) + 1e-6)
        close(unit(out.cpu().double().reshape(T, heads, vdim)), unit(want), dtype, f"matrix memory, call {call}", f32=2e-4, bf16=3e-2)
        got = state[:, : heads * per_head].cpu().double().reshape(8, heads, per_head)
        close(got[:, :, : dim * vdim].reshape(8, heads, dim, vdim), S, torch.float32, f"its S, call {call}", f32=2e-4)
        close(got[:, :, dim * vdim : dim * vdim + dim], N, torch.float32, f"its n, call {call}", f32=2e-4)
        close(got[:, :, -1], M, torch.float32, f"its m, call {call}")
    assert float(state[:, heads * per_head :].abs().max()) == 0.0
    assert float(state[7].abs().max()) == 0.0
