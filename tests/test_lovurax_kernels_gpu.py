"""The kernels of the Lovurax parts on the device against plain formulas in float64: the retention's rotation and its scan (walked
a row at a time and cut into chunks that run side by side, over rows of unequal length, from states that an earlier call left),
the attention with sigmoid weights (prepared heads, cache entries of one plane and of two, splits), the xIELU activation, the gate
a head, and the gated sum into the 32-bit stream with its norm."""
import math

import pytest
import torch

from tests import helpers as H
from tests.plain import lovurax_plain as P

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
@pytest.mark.parametrize("heads,dim,rot", [(2, 8, 4), (3, 64, 64), (1, 160, 32), (2, 6, 0)])
def test_the_retention_rotation(kernels, dtype, heads, dim, rot):
    g = torch.Generator().manual_seed(dim)
    T = 37
    u = torch.randn(T, 2 * heads * dim + 11, generator=g).to(dtype)        # other columns follow and are not read
    positions = torch.randint(0, 5000, (T,), generator=g).to(torch.int32)
    inv_freq = torch.tensor([777.0 ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float64) if rot else None
    qk = kernels.retention_prepare(u.cuda(), inv_freq.cuda() if rot else None, rot, positions.cuda(), heads, dim, dim ** -0.5)
    x = u[:, : 2 * heads * dim].double().reshape(T, 2 * heads, dim)
    want = P.rotate_halves(x, positions, rot, 777.0) if rot else x.clone()
    want[:, heads:] *= dim ** -0.5
    close(qk.cpu(), want.reshape(T, -1), torch.float32, "retention rotation", f32=1e-5)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,dim,vdim", [(2, 20, 36), (1, 64, 70), (3, 100, 32), (1, 160, 40), (1, 520, 33)])
@pytest.mark.parametrize("chunked", [False, True])
def test_the_retention_scan_walked_and_in_chunks(kernels, dtype, heads, dim, vdim, chunked):
    g = torch.Generator().manual_seed(heads * dim + vdim)
    T = sum(ROWS)
    r = lambda *shape: torch.randn(*shape, generator=g)
    slots = [5, 0, 3, 1, 6, 2, 4]
    indptr = [0]
    for n in ROWS:
        indptr.append(indptr[-1] + n)
    decay = torch.tensor([0.0, 0.97, 1.0][:heads] if heads > 1 else [0.99], dtype=torch.float32)
    per = heads * dim * vdim
    state = torch.zeros(8, per + 3).cuda()                          # a slot wider than the state: the stride is the slot's
    S = torch.zeros(8, heads, dim, vdim, dtype=torch.float64)
    v_col = 5
    for call in range(2):                                          # the second call starts from what the first one left
        qk = (r(T, 2 * heads * dim) * dim ** -0.25).float()
        u = r(T, v_col + heads * vdim + 2).to(dtype)
        out = kernels.retention_scan(qk.cuda(), u.cuda(), v_col, state, decay.cuda(), i32(indptr), i32(slots), heads, dim, vdim, chunked=chunked)
        q = qk[:, : heads * dim].double().reshape(T, heads, dim)
        k = qk[:, heads * dim :].double().reshape(T, heads, dim)
        v = u[:, v_col : v_col + heads * vdim].double().reshape(T, heads, vdim)
        want = torch.zeros(T, heads, vdim, dtype=torch.float64)
        for row, slot in enumerate(slots):
            for t in range(indptr[row], indptr[row + 1]):
                S[slot] = decay.double()[:, None, None] * S[slot] + k[t][:, :, None] * v[t][:, None, :]
                want[t] = torch.einsum("hdv,hd->hv", S[slot], q[t])
        close(out.cpu().reshape(T, heads, vdim), want, torch.float32, f"retention, call {call}", f32=1e-4)
        close(state[:, :per].cpu().reshape(8, heads, dim, vdim), S, torch.float32, f"its state, call {call}", f32=1e-4)
    assert float(state[:, per:].abs().max()) == 0.0                 # nothing written beside the state
    assert float(state[7].abs().max()) == 0.0                       # nor into a slot no row names


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("gate", ["sigmoid", "silu"])
def test_the_head_norm_with_and_without_a_weight(kernels, dtype, gate):
    g = torch.Generator().manual_seed(3)
    T, heads, vdim, col = 9, 3, 20, 7
    o = torch.randn(T, heads * vdim, generator=g)
    u = torch.randn(T, col + heads * vdim, generator=g).to(dtype)
    for w in (None, 1.0 + 0.2 * torch.randn(heads * vdim, generator=g)):
        got = kernels.head_norm_gate(o.cuda(), u.cuda(), col, None if w is None else w.cuda(), heads, 1e-5, dtype, gate=gate)
        x = P.rms_norm(o.double().reshape(T, heads, vdim), None, 1e-5).reshape(T, -1)
        z = u[:, col:].double()
        want = x * (1.0 if w is None else w.double()) * P.sigmoid(z) * (z if gate == "silu" else 1.0)
        close(got.cpu(), want, dtype, f"head norm, gate {gate}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,dim,vdim", [(4, 2, 8, 6), (3, 3, 48, 48), (9, 1, 20, 33), (2, 1, 128, 64), (4, 2, 64, 64), (2, 2, 32, 128), (4, 1, 128, 128)])
def test_the_attention_with_sigmoid_weights(kernels, dtype, heads, kv_heads, dim, vdim):
    """Two rows of unequal length whose pages lie scattered in the pool, keys written by the prepare kernel in two calls (a prompt's
    portion, then the rest), queries at every position; a small bound on the lengths makes the kernel deal a token's keys to
    several blocks, a large one to one."""
    g = torch.Generator().manual_seed(heads * dim + vdim)
    page, eps, scale, coef, every = 4, 1e-5, 0.7 / math.sqrt(dim), 0.4, 7
    lens = [45, 150]
    T = sum(lens)
    width = (heads + kv_heads) * dim + kv_heads * vdim
    qkv = torch.randn(T, width + heads * vdim, generator=g).to(dtype)             # the output gate's columns follow
    q_w, k_w = 1.0 + 0.2 * torch.randn(dim, generator=g), 1.0 + 0.2 * torch.randn(dim, generator=g)
    slopes = torch.tensor(P.head_slopes(heads), dtype=torch.float32)
    bias = -1.0 + torch.randn(heads, generator=g)
    pages_of = [torch.randperm(40, generator=g)[:12].tolist(), (40 + torch.randperm(40, generator=g)[:38]).tolist()]
    two_planes = dim == vdim
    pool = torch.zeros((2 if two_planes else 1, 80, kv_heads, page, dim if two_planes else dim + vdim), dtype=dtype).cuda()
    k_pool, v_pool = pool[0], (pool[1] if two_planes else None)
    positions = torch.cat([torch.arange(n) for n in lens]).to(torch.int32)
    token_row = torch.cat([torch.full((n,), i) for i, n in enumerate(lens)]).to(torch.int32)
    slot_mapping = torch.tensor([pages_of[int(r)][int(p) // page] * page + int(p) % page for r, p in zip(token_row, positions)], dtype=torch.int32)
    kv_indptr, kv_indices = i32([0, 12, 50]), i32(pages_of[0] + pages_of[1])
    dev = qkv.cuda()
    first = torch.cat([torch.arange(0, 20), torch.arange(45, 45 + 33)])             # each row's first portion, then the rest
    rest = torch.tensor([t for t in range(T) if t not in set(first.tolist())])
    q = torch.zeros(T, heads, dim, dtype=dtype).cuda()
    for part in (first, rest):
        q[part] = kernels.sigmoid_attention_prepare(dev[part].contiguous(), k_pool, v_pool, q_w.cuda(), k_w.cuda(), positions[part].cuda(),
                                                    slot_mapping[part].cuda(), heads, kv_heads, dim, vdim, eps, coef, every, page)
    x = qkv.double()
    Q, K = heads * dim, kv_heads * dim
    temp = torch.tensor([1.0 + coef * math.log((int(p) + 1) // every + 1) for p in positions], dtype=torch.float64)
    rd = lambda t: t.to(dtype).double()
    qn = rd(P.rms_norm(x[:, :Q].reshape(T, heads, dim), q_w.double(), eps) * temp[:, None, None])
    kn = rd(P.rms_norm(x[:, Q : Q + K].reshape(T, kv_heads, dim), k_w.double(), eps))
    v = x[:, Q + K : width].reshape(T, kv_heads, vdim)
    close(q.cpu(), qn, dtype, "prepared queries", bf16=1e-2)
    want = torch.zeros(T, heads, vdim, dtype=torch.float64)
    group = heads // kv_heads
    for t in range(T):
        row, p = int(token_row[t]), int(positions[t])
        start = t - p
        for h in range(heads):
            s = (kn[start : t + 1, h // group] @ qn[t, h]) * scale - float(slopes[h]) * (p - torch.arange(p + 1, dtype=torch.float64)) + float(bias[h])
            want[t, h] = P.sigmoid(s) @ v[start : t + 1, h // group]
    gated = want.reshape(T, -1) * P.sigmoid(x[:, width:])
    for kv_cap in (0, 160, 4096):        # a bound on the rows' lengths (0: none given)
        got = kernels.sigmoid_attention(q, k_pool, v_pool, dev, width, slopes.cuda(), bias.cuda(), positions.cuda(), token_row.cuda(), kv_indptr,
                                        kv_indices, kv_heads, vdim, scale, kv_cap=kv_cap)
        close(got.cpu(), gated, dtype, f"sigmoid attention with its gate, bound {kv_cap}")
    got = kernels.sigmoid_attention(q, k_pool, v_pool, None, None, slopes.cuda(), bias.cuda(), positions.cuda(), token_row.cuda(), kv_indptr, kv_indices,
                                    kv_heads, vdim, scale, kv_cap=160)
    close(got.cpu(), want.reshape(T, -1), dtype, "sigmoid attention without a gate")
    # a step of few tokens deals every token's keys to several blocks: the last tokens of both rows and two in between
    few = torch.tensor([31, 44, 45, 45 + 63, 45 + 64, T - 1])
    for kv_cap in (160, 1024, 96):       # the last: a bound the second row exceeds
        got = kernels.sigmoid_attention(q[few.cuda()].contiguous(), k_pool, v_pool, dev[few.cuda()].contiguous(), width, slopes.cuda(), bias.cuda(),
                                        positions[few].cuda(), token_row[few].cuda(), kv_indptr, kv_indices, kv_heads, vdim, scale, kv_cap=kv_cap)
        close(got.cpu(), gated[few], dtype, f"sigmoid attention of few tokens, bound {kv_cap}")
    if dtype == torch.bfloat16 and kernels.sigmoid_attention_mma_supported(dim, vdim, two_planes):
        # the tensor-core form: rows of 45 and 150 tokens are one and three tiles of queries over up to three tiles of keys
        q_indptr = i32([0, lens[0], T])
        for rows, col in ((dev, width), (None, None)):
            got = kernels.sigmoid_attention(q, k_pool, v_pool, rows, col, slopes.cuda(), bias.cuda(), positions.cuda(), token_row.cuda(), kv_indptr,
                                            kv_indices, kv_heads, vdim, scale, kv_cap=160, q_indptr=q_indptr)
            close(got.cpu(), gated if rows is not None else want.reshape(T, -1), dtype, "sigmoid attention on the tensor cores")
        # a long row's keys dealt to several blocks in chunks of one and of two tiles of 64 keys (the kernel's own chunk is longer than
        # these rows): the second row's later queries have two and three chunks, the first row's one
        kept = kernels.SIGMOID_MMA_CHUNK_TILES
        try:
            for tiles, kv_cap in ((1, 1024), (2, 1024), (1, 64)):      # the last: a bound the second row exceeds (two chunks for three tiles)
                kernels.SIGMOID_MMA_CHUNK_TILES = tiles
                got = kernels.sigmoid_attention(q, k_pool, v_pool, dev, width, slopes.cuda(), bias.cuda(), positions.cuda(), token_row.cuda(), kv_indptr,
                                                kv_indices, kv_heads, vdim, scale, kv_cap=kv_cap, q_indptr=q_indptr)
                close(got.cpu(), gated, dtype, f"sigmoid attention on the tensor cores, chunks of {tiles} tiles under a bound of {kv_cap}")
        finally:
            kernels.SIGMOID_MMA_CHUNK_TILES = kept


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n", [(5, 7), (33, 64), (1, 4096)])
def test_xielu(kernels, dtype, n):
    g = torch.Generator().manual_seed(n[1])
    x = (3.0 * torch.randn(*n, generator=g)).to(dtype)
    p, q = torch.tensor(0.3, dtype=torch.float64), torch.tensor(-0.8, dtype=torch.float64)
    got = kernels.xielu(x.cuda(), float(P.softplus(p)), 0.5 + float(P.softplus(q)))
    close(got.cpu(), P.xielu(x.double(), p, q), dtype, "xielu", f32=1e-6, bf16=8e-3)


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_gate_a_head_and_scaled_logits(kernels, dtype):
    g = torch.Generator().manual_seed(5)
    T, heads, vdim, col = 13, 5, 12, 3
    x = torch.randn(T, heads * vdim, generator=g).to(dtype)
    gate = torch.randn(T, col + heads + 2, generator=g).to(dtype)
    got = kernels.head_gate_mul_(x.cuda(), gate.cuda(), col, heads)
    want = (x.double().reshape(T, heads, vdim) * P.sigmoid(gate[:, col : col + heads].double())[:, :, None]).reshape(T, -1)
    close(got.cpu(), want, dtype, "gate a head")
    logits = torch.randn(7, 301, generator=g)
    close(kernels.scale_(logits.clone().cuda(), 0.37).cpu(), logits.double() * 0.37, torch.float32, "scaled logits", f32=1e-6)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden", [40, 192, 2048])
def test_the_gated_sum_into_the_stream_and_its_norm(kernels, dtype, hidden):
    g = torch.Generator().manual_seed(hidden)
    T, eps = 11, 1e-5
    stream = torch.randn(T, hidden, generator=g)
    y = torch.randn(T, hidden, generator=g).to(dtype)
    arguments, bias, w = 2.0 * torch.randn(T, hidden, generator=g), torch.randn(hidden, generator=g), 1.0 + 0.1 * torch.randn(hidden, generator=g)
    total = stream.double() + y.double() * P.sigmoid(arguments.double() + bias.double())
    dev = stream.clone().cuda()
    rows = i32([9, 0, 4])
    got = kernels.wide_rms_norm_gated(dev, w.cuda(), eps, dtype, y.cuda(), arguments.cuda(), bias.cuda(), rows)
    close(got.cpu(), P.rms_norm(total[[9, 0, 4]], w.double(), eps), dtype, "gated sum and norm of gathered rows")
    assert torch.equal(dev.cpu(), stream)                             # gathered rows leave the stream as it was
    got = kernels.wide_rms_norm_gated(dev, w.cuda(), eps, dtype, y.cuda(), arguments.cuda(), bias.cuda())
    close(got.cpu(), P.rms_norm(total, w.double(), eps), dtype, "gated sum and norm")
    close(dev.cpu(), total, torch.float32, "the stream after the sum", f32=1e-6)


@pytest.mark.parametrize("heads,dim,vdim,width", [(3, 16, 48, 24), (2, 64, 64, 256), (1, 128, 32, 40), (4, 32, 128, 64)])
def test_prompt_portions_over_keys_and_values_carried_out_of_a_latent_cache(kernels, heads, dim, vdim, width):
    """The gather of two rows' cached vectors from scattered pages into dense stretches (zeros beyond a row), and the causal softmax
    attention over keys and values laid out that way: rows of 45 and 150 tokens whose queries are the second row's last 100 tokens and
    all of the first row's, so that a row's queries start inside its keys."""
    g = torch.Generator().manual_seed(heads * dim + vdim)
    page, stride, scale = 4, 192, 1.3 / math.sqrt(dim)
    lens = [45, 150]
    pages_of = [torch.randperm(40, generator=g)[:12].tolist(), (40 + torch.randperm(40, generator=g)[:38]).tolist()]
    pool = torch.randn(80, 1, page, width, generator=g).to(torch.bfloat16).cuda()
    kv_indptr, kv_indices = i32([0, 12, 50]), i32(pages_of[0] + pages_of[1])
    latents = kernels.latent_gather(pool, i32(lens), kv_indptr, kv_indices, 2, stride)
    want = torch.zeros(2 * stride, width, dtype=torch.bfloat16)
    for r, n in enumerate(lens):
        for j in range(n):
            want[r * stride + j] = pool[pages_of[r][j // page], 0, j % page].cpu()
    assert torch.equal(latents.cpu(), want)
    keys = torch.randn(2 * stride, heads * dim, generator=g).to(torch.bfloat16)
    values = torch.randn(2 * stride, heads * vdim, generator=g).to(torch.bfloat16)
    starts = [0, 50]                                   # the first position each row brings queries for
    positions = torch.cat([torch.arange(s0, n) for s0, n in zip(starts, lens)]).to(torch.int32)
    T = positions.numel()
    q = torch.randn(T, heads * dim + 8, generator=g).to(torch.bfloat16)         # other columns follow a token's queries
    q_indptr = i32([0, lens[0] - starts[0], T])
    got = kernels.carried_attention(q.cuda(), keys.cuda(), values.cuda(), positions.cuda(), q_indptr, heads, dim, vdim, stride, scale)
    ref = torch.zeros(T, heads, vdim, dtype=torch.float64)
    t = 0
    for r, (s0, n) in enumerate(zip(starts, lens)):
        K = keys[r * stride : r * stride + n].double().reshape(n, heads, dim)
        V = values[r * stride : r * stride + n].double().reshape(n, heads, vdim)
        for p in range(s0, n):
            for h in range(heads):
                w = torch.softmax((K[: p + 1, h] @ q[t, h * dim : (h + 1) * dim].double()) * scale, dim=0)
                ref[t, h] = w @ V[: p + 1, h]
            t += 1
    close(got.cpu(), ref.reshape(T, -1), torch.bfloat16, "attention over carried keys and values")
