"""The Nomivik decoder through the engine's step function, cache manager, scheduler and entry point, against the plain
implementation of tests/plain/nomivik_plain.py, for every way of cutting the work.

Each test runs on the GPU with the real kernel library in float32 (captured steps) and bfloat16 (marked gpu), and on the
CPU with the stand-in kernels of tests/fake_kernels.py, which checks the host side: the batch tables, the pages and slots, the
previous token a request keeps, the order of the layer runs and which state each pass of a looped range gets.
"""
import copy
import random

import pytest
import torch

from roost_b200 import GenerationOptions, RoostEngine
from roost_b200.config.nomivik import NomivikConfig
from roost_b200.config.reader import ConfigError, ConfigReader
from roost_b200.engine.executor import StepEntry, StepExecutor
from roost_b200.weights.loader import WeightError
from tests import helpers as H
from tests import nomivik_models as NM
from tests.plain import nomivik_plain as P

BACKENDS = [
    pytest.param(("gpu", torch.float32), id="gpu-f32", marks=pytest.mark.gpu),
    pytest.param(("gpu", torch.bfloat16), id="gpu-bf16", marks=pytest.mark.gpu),
    pytest.param(("fake", torch.float32), id="cpu-fake"),
]
# Two bounds: the root-mean-square error of all logits of a request, and the largest root-mean-square error of one position's
# logits (both relative to the logits' own root mean square). A fault that strikes one position (a key lost at a window's edge,
# a wrong page or slot in one step, a previous token taken from another request) moves that position's logits by tens of
# percent and barely shows among hundreds of positions; rounding alone stays far below both bounds.
F32_TOKEN, F32_RMS = 1e-3, 3e-5
BF16_TOKEN, BF16_RMS = 0.3, 0.06


@pytest.fixture(params=BACKENDS)
def backend(request):
    return request.param


_MODELS: dict = {}


def model_dir(tmp_path_factory, name, cfg, seed, change=None):
    """A model folder written once a session; ``change(cfg, tensors)`` edits the drawn weights first."""
    if name not in _MODELS:
        tensors = NM.draw_tensors(cfg, seed)
        if change is not None:
            change(cfg, tensors)
        _MODELS[name] = (NM.write_model(tmp_path_factory.mktemp(f"nomivik_{name}"), cfg, tensors), cfg, NM.plain_weights(tensors))
    return _MODELS[name]


class Run:
    """Drives a StepExecutor and keeps, per request, the logits of every position."""

    def __init__(self, model_dir, cfg, backend, page_size=4, num_pages=64, slots=4, graphs=True):
        kind, self.dtype = backend
        self.cfg = cfg
        self.model = H.make_model(model_dir, self.dtype, kind)
        self.ex = StepExecutor(self.model, page_size=page_size, num_pages=num_pages, max_requests=slots, use_graphs=graphs)
        self.logits: dict = {}

    def step(self, entries):
        """entries: [(request id, tokens)]; every position's logits are asked for."""
        out = self.ex.step([StepEntry(rid, list(toks), list(range(len(toks)))) for rid, toks in entries])
        at = 0
        for rid, toks in entries:
            self.logits.setdefault(rid, []).append(out[at : at + len(toks)].float().cpu())
            at += len(toks)
        self.ex.cache.check_invariants()

    def finish(self, rid):
        self.ex.finish(rid)

    def check(self, rid, ids, weights, what, bf16_bounds=(BF16_TOKEN, BF16_RMS), f32_bounds=(F32_TOKEN, F32_RMS)):
        got = torch.cat(self.logits.pop(rid))
        want = P.forward(self.cfg, weights, list(ids[: got.shape[0]]))
        worst, bound = f32_bounds if self.dtype == torch.float32 else bf16_bounds
        keep = torch.ones(got.shape[0], dtype=torch.bool)
        if self.dtype != torch.float32:
            # Positions where rounding every norm's and projection's output to 16 bits moves the plain logits far by itself
            # (the matrix memory's output keeps only the direction of S^T q, and when one token holds the memory that
            # direction hangs on the sign of one dot product, which can lie next to zero) are ill-conditioned, not faulty:
            # they are left out in 16 bits, and the 32-bit run of the same kernels checks them.
            rounded = P.forward(self.cfg, weights, list(ids[: got.shape[0]]), rounding=lambda z: z.to(torch.bfloat16).double())
            keep = position_errors(rounded, want) < worst / 3
            assert int((~keep).sum()) <= max(3, got.shape[0] // 10), f"{what}: the test's model is ill-conditioned at {int((~keep).sum())} positions"
        err, rms = float(position_errors(got, want)[keep].max()), H.rms_error(got[keep], want[keep])
        print(f"MEASURED {what} {self.dtype}: worst position's error {err:.3e}, rms error {rms:.3e}, {int((~keep).sum())} positions left out")
        assert err < worst and rms < bound, f"{what}: worst position's error {err}, rms error {rms}"
        return got, want

    def all_free(self):
        return all(p.used_count == 0 for p in self.ex.cache.pools)


def position_errors(got, want):
    """Every position's error: root mean square of its logits' differences over that of its logits."""
    got, want = got.double().cpu(), want.double().cpu()
    return (got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean(-1).sqrt()


def token_error(got, want) -> float:
    return float(position_errors(got, want).max())


def ids_for(cfg, n, seed):
    return H.random_ids(n, cfg["vocab"], seed)


# One mechanism a model, so that a fault names its mechanism.
SINGLE = {
    "recurrence_only": NM.config([(NM.recurrence(width=14, blocks=2, conv=4), None)], width=20, vocab=45, side=None, pairs=None),
    "attention_and_memory": NM.config([(NM.parallel(NM.attention(heads=2, kv_heads=2, dim=6, vdim=5, rot=6, window=5), NM.memory(heads=1, dim=4, vdim=7)), None)],
                                      width=24, vocab=50, side=None, pairs=None),
    "pairs_only": NM.config([(NM.recurrence(width=8, blocks=1, conv=2), None)], width=16, vocab=30, side=None, pairs=(11, 5, 3)),
    "token_input_only": NM.config([(NM.recurrence(width=8, blocks=2, conv=2), None), (NM.recurrence(width=6, blocks=3, conv=3), None)], width=16, vocab=31,
                                  side=3, pairs=None),
    "dense_after_parallel": NM.config([(NM.parallel(), NM.dense(ff=17))], width=28, vocab=33, side=None, pairs=None),
    "looped_pair": NM.config([(NM.parallel(NM.attention(heads=2, kv_heads=1, dim=4, vdim=4, rot=2, window=3), NM.memory(heads=2, dim=3, vdim=3)), None),
                              (NM.recurrence(width=8, blocks=4, conv=2), None)], width=16, vocab=30, side=2, loop=(0, 2, 3)),
}
ALL = dict(NM.CONFIGS, **SINGLE)


@pytest.fixture(params=sorted(ALL))
def any_model(request, tmp_path_factory):
    return (request.param,) + model_dir(tmp_path_factory, request.param, ALL[request.param], seed=len(request.param))


@pytest.fixture(params=sorted(NM.CONFIGS))
def model(request, tmp_path_factory):
    return (request.param,) + model_dir(tmp_path_factory, request.param, NM.CONFIGS[request.param], seed=len(request.param))


# ------------------------------------------------------------------------------------------------ whole prompts
@pytest.mark.parametrize("length", [1, 2, 3, 37, 150])
def test_each_mechanism_and_each_model_on_whole_prompts(any_model, backend, length):
    """Models of one mechanism each and the mixed models; the shortest prompts are the first tokens of a sequence: the pair
    table's last row, the convolution's zeros before the start, empty states, a running maximum that starts at zero, a softmax
    over one key and the sink."""
    name, folder, cfg, weights = any_model
    run = Run(folder, cfg, backend)
    ids = ids_for(cfg, length, seed=length)
    run.step([("r", ids)])
    run.finish("r")
    run.check("r", ids, weights, f"{name} whole {length}")
    assert run.all_free()


def test_the_residual_after_every_layer_run(model, backend):
    """The engine's stream after every run of a layer (a looped layer counts each time) against the plain one."""
    name, folder, cfg, weights = model
    kind, dtype = backend
    m = H.make_model(folder, dtype, kind)
    ex = StepExecutor(m, page_size=4, num_pages=32, max_requests=2, use_graphs=False)
    ids = ids_for(cfg, 21, seed=9)
    seen = []

    class Watched:
        """A block that notes the stream it leaves: the 32-bit residual plus the branch output still to be added."""

        def __init__(self, block):
            self.block = block

        def __getattr__(self, name):
            return getattr(self.block, name)

        def __call__(self, *args, **kwargs):
            a, residual = self.block(*args, **kwargs)
            seen.append((residual.float() + a.float()).cpu())
            return a, residual

    m.blocks = [Watched(b) for b in m.blocks]
    ex.step([StepEntry("r", ids, [20])])
    want = []
    P.forward(cfg, weights, ids, collect=want)
    assert len(seen) == len(want) == len(P.layer_order(cfg))
    for i, (g, w) in enumerate(zip(seen, want)):
        err = H.rms_error(g, w)
        assert err < (2e-5 if dtype == torch.float32 else 0.03), f"{name}: the stream after layer run {i} differs by {err}"


# ------------------------------------------------------------------------------------------------ cutting the work
def test_prefill_against_token_by_token_decoding(model, backend):
    name, folder, cfg, weights = model
    run = Run(folder, cfg, backend)
    ids = ids_for(cfg, 70, seed=5)
    for head in (0, 1, 38):     # from the very first token on; after one token; after a prompt that ends inside a page
        rid = f"r{head}"
        if head:
            run.step([(rid, ids[:head])])
        for t in ids[head:]:
            run.step([(rid, [t])])
        run.finish(rid)
        run.check(rid, ids, weights, f"{name} decoded from {head}")
    assert run.all_free()


@pytest.mark.parametrize("sizes", [[2, 3, 2, 5, 7, 16, 33], [33, 2, 2, 1, 9], [1, 2]])
def test_portions_of_several_sizes_down_to_two_tokens(model, backend, sizes):
    """A portion's first token takes its pair row from the request's previous token, its convolution from the taps the
    state kept, its recurrences and memories from the slot, and its window reaches back into earlier portions."""
    name, folder, cfg, weights = model
    run = Run(folder, cfg, backend)
    ids = ids_for(cfg, 90 if len(sizes) > 2 else 25, seed=sum(sizes))
    at, i = 0, 0
    while at < len(ids):
        n = min(sizes[i % len(sizes)], len(ids) - at)
        run.step([("r", ids[at : at + n])])
        at, i = at + n, i + 1
    run.finish("r")
    run.check("r", ids, weights, f"{name} portions {sizes}")


def test_batches_of_unequal_requests_with_pages_and_slots_used_again(model, backend):
    """Six requests of unequal length through three state slots and a pool of pages that holds three of them: portions
    of some beside single tokens of others; a request may sit out a step; a request that ends gives its pages and slot
    to the next one, whose states must start empty and whose first token must take the pair table's last row."""
    name, folder, cfg, weights = model
    run = Run(folder, cfg, backend, page_size=4, num_pages=48, slots=3)
    rng = random.Random(11)
    reqs = {f"q{i}": ids_for(cfg, n, seed=20 + i) for i, n in enumerate([41, 9, 64, 23, 2, 55])}
    waiting, live = list(reqs), {}
    slots_seen = set()
    while waiting or live:
        while waiting and len(live) < 3:
            live[waiting.pop(0)] = 0
        entries = []
        for rid in [r for r in live if rng.random() < 0.8] or [next(iter(live))]:
            left = len(reqs[rid]) - live[rid]
            n = 1 if left <= 6 else min(left - 6, rng.choice([2, 3, 5, 8, 17]))
            entries.append((rid, reqs[rid][live[rid] : live[rid] + n]))
            live[rid] += n
        run.step(entries)
        for gi, g in enumerate(run.ex.groups):
            if g.kind == "state" and g.runs:
                slots_seen.update(run.ex.cache.get(rid).slots[gi] for rid, _ in entries)
        for rid, _ in entries:
            if live[rid] == len(reqs[rid]):
                run.finish(rid)
                del live[rid]
    assert slots_seen <= {0, 1, 2}
    for rid, ids in reqs.items():
        run.check(rid, ids, weights, f"{name} mixed {rid}")
    assert run.all_free()


def test_a_batch_gives_each_request_what_it_gets_alone(model, backend):
    """The same three requests alone and side by side in one batch, cut the same way: beyond rounding nothing may differ."""
    name, folder, cfg, weights = model
    reqs = {f"s{i}": ids_for(cfg, n, seed=40 + i) for i, n in enumerate([33, 7, 50])}
    cuts = {"s0": [20, 2, 11], "s1": [1, 1, 5], "s2": [2, 40, 8]}
    alone = Run(folder, cfg, backend)
    for rid, ids in reqs.items():
        at = 0
        for n in cuts[rid]:
            alone.step([(rid, ids[at : at + n])])
            at += n
        alone.finish(rid)
    together = Run(folder, cfg, backend)
    at = {rid: 0 for rid in reqs}
    for step in range(3):
        together.step([(rid, reqs[rid][at[rid] : at[rid] + cuts[rid][step]]) for rid in reqs])
        for rid in reqs:
            at[rid] += cuts[rid][step]
    for rid in reqs:
        a, b = torch.cat(alone.logits[rid]), torch.cat(together.logits[rid])
        err = token_error(b, a)
        assert err < (2e-5 if backend[1] == torch.float32 else 0.1), f"{name} {rid}: alone and in a batch differ by {err}"


def test_long_decoding_over_many_pages(model, backend):
    """230 tokens one by one: every window of the models passes over decoded tokens, pages behind a window are given back
    where the cache manager does that, states are carried 227 times."""
    name, folder, cfg, weights = model
    run = Run(folder, cfg, backend, page_size=4, num_pages=80)
    ids = ids_for(cfg, 230, seed=3)
    run.step([("r", ids[:3])])
    for t in ids[3:]:
        run.step([("r", [t])])
    run.finish("r")
    run.check("r", ids, weights, f"{name} long decoding")


LONG = NM.config([(NM.parallel(NM.attention(heads=4, kv_heads=2, dim=16, vdim=24, rot=8, base=10000.0, scale=0.25, window=200),
                               NM.memory(heads=2, dim=20, vdim=36, gate_cap=8.0)), NM.dense(ff=128)),
                  (NM.recurrence(width=48, blocks=4, conv=4), NM.dense(ff=256))], width=72, vocab=83, pairs=(101, 13, 17), side=7)


def test_a_long_prompt_takes_the_forms_of_steps_of_many_rows(tmp_path_factory, backend):
    """700 tokens in one step and then 2 + 1: the kernels' forms for many tokens a row (the recurrences cut into chunks where
    they are) and a window that ends far inside the prompt."""
    folder, cfg, weights = model_dir(tmp_path_factory, "long", LONG, seed=21)
    run = Run(folder, cfg, backend, page_size=16, num_pages=64)
    ids = ids_for(cfg, 703, seed=8)
    run.step([("r", ids[:700])])
    run.step([("r", ids[700:702])])
    run.step([("r", ids[702:])])
    run.finish("r")
    run.check("r", ids, weights, "long prompt")


def test_the_first_tokens_of_a_sequence_one_by_one(any_model, backend):
    """A request decoded from its very first token: the pair table's last row, one key and the sink, empty states, a running
    maximum of zero, zeros before the convolution."""
    name, folder, cfg, weights = any_model
    run = Run(folder, cfg, backend)
    ids = ids_for(cfg, 6, seed=1)
    for t in ids:
        run.step([("r", [t])])
    run.finish("r")
    run.check("r", ids, weights, f"{name} first tokens")


# ------------------------------------------------------------------------------------------------ keys that must, or must not, be seen
KEY, QUERY = 7, 11        # token ids: QUERY scores KEY far above every other key in the first layer's attention
WINDOW = 37               # no multiple of a page of four, of a tile of 32 keys or of anything else
# Only the first layer's attention can carry the key token to the query token here: the matrix memory beside it gets a large
# negative input gate (below) and there is no recurrence, so whether the key is inside the window decides the logits.
EDGE = NM.config([(NM.parallel(NM.attention(heads=2, kv_heads=1, dim=16, vdim=6, rot=2, scale=0.9, window=WINDOW, softcap=30.0), NM.memory(heads=1, dim=4, vdim=4, gate_cap=20.0)), None),
                  (NM.parallel(NM.attention(heads=2, kv_heads=2, dim=4, vdim=4, rot=4, window=1, softcap=5.0), NM.memory(heads=1, dim=3, vdim=5, gate_cap=20.0)), NM.dense(ff=16))],
                 width=32, vocab=53, pairs=(41, 7, 3), side=4)
FAR = NM.config([(NM.parallel(NM.attention(heads=2, kv_heads=1, dim=32, vdim=6, rot=2, scale=0.5, window=400, softcap=30.0), NM.memory(heads=1, dim=4, vdim=4, gate_cap=20.0)), None),
                 (NM.recurrence(width=8, blocks=2, conv=2), NM.dense(ff=16))], width=32, vocab=53, pairs=(41, 7, 3), side=4)


def sharpened(tmp_path_factory, name, cfg):
    def change(c, t):
        NM.sharpen(c, t, KEY, QUERY)
        for i, layer in enumerate(c["layers"]):
            if layer["type"] == "parallel":        # a memory that takes in next to nothing: exp(i - m) with i near -20
                t[f"l{i}.mix.right.i.b"] = torch.full_like(t[f"l{i}.mix.right.i.b"], -60.0)
                t[f"l{i}.mix.right.i"] = torch.zeros_like(t[f"l{i}.mix.right.i"])
    return model_dir(tmp_path_factory, name, cfg, seed=77, change=change)


def filler(cfg, n, seed):
    rng = random.Random(seed)
    return [rng.choice([t for t in range(cfg["vocab"]) if t not in (KEY, QUERY)]) for _ in range(n)]


@pytest.mark.parametrize("decoded", [False, True], ids=["in a prompt", "decoded"])
def test_a_key_just_inside_and_just_outside_the_window(tmp_path_factory, backend, decoded):
    """The key token sits window - 2, window - 1 (the last place the window keeps), window and window + 1 places before the
    query token, with the query at several offsets of a page, in a prompt cut in two and decoded token by token. The plain
    logits of the query's position with the key inside differ from those with it outside by far more than the bound (the
    test checks that), so a window that is one token off fails one side or the other."""
    folder, cfg, weights = sharpened(tmp_path_factory, "edge", EDGE)
    run = Run(folder, cfg, backend, page_size=4, num_pages=120)
    for query_at in (90, 91, 92, 93, 128):
        seen = {}
        for gap in (None, WINDOW - 2, WINDOW - 1, WINDOW, WINDOW + 1):
            ids = filler(cfg, query_at + 6, seed=query_at)
            if gap is not None:
                ids[query_at - gap] = KEY
            ids[query_at] = QUERY
            rid = f"edge{query_at}_{gap}"
            if decoded:
                run.step([(rid, ids[: query_at - 50])])
                for t in ids[query_at - 50 :]:
                    run.step([(rid, [t])])
            else:
                run.step([(rid, ids[: query_at - 20])])
                run.step([(rid, ids[query_at - 20 :])])
            run.finish(rid)
            got, want = run.check(rid, ids, weights, f"query at {query_at}, key {gap} back")
            seen[gap] = (got[query_at], want[query_at])
        for gap in (WINDOW - 2, WINDOW - 1):
            assert H.rms_error(seen[gap][1][None], seen[None][1][None]) > 2 * BF16_TOKEN          # the test's own sharpness
            assert H.rms_error(seen[gap][0][None], seen[None][0][None]) > BF16_TOKEN              # the engine saw the key
        for gap in (WINDOW, WINDOW + 1):
            assert H.rms_error(seen[gap][1][None], seen[WINDOW - 1][1][None]) > 2 * BF16_TOKEN
            assert H.rms_error(seen[gap][0][None], seen[WINDOW - 1][0][None]) > BF16_TOKEN        # the engine did not


@pytest.mark.parametrize("decoded", [False, True], ids=["in a prompt", "decoded"])
def test_a_key_far_away_among_hundreds_at_every_page_offset(tmp_path_factory, backend, decoded):
    """The key token sits 288 to 321 places before the query token, inside a window of 400, once at every offset of a page of
    four and across the borders of the 32-key tiles; losing that one key (a wrong page, a tile's or a split's edge) changes the
    query's logits by far more than the bound."""
    folder, cfg, weights = sharpened(tmp_path_factory, "far", FAR)
    run = Run(folder, cfg, backend, page_size=4, num_pages=120)
    seen = {}
    for at in (None, 0, 1, 2, 3, 31, 32, 33):
        ids = filler(cfg, 330, seed=4)
        if at is not None:
            ids[at] = KEY
        ids[321] = QUERY
        rid = f"far{at}"
        if decoded:
            run.step([(rid, ids[:300])])
            for t in ids[300:]:
                run.step([(rid, [t])])
        else:
            run.step([(rid, ids[:130])])
            run.step([(rid, ids[130:])])
        run.finish(rid)
        got, want = run.check(rid, ids, weights, f"far key at {at}")
        seen[at] = want[321]
    for at in (0, 1, 2, 3, 31, 32, 33):
        moved = H.rms_error(seen[at][None], seen[None][None])
        print(f"MEASURED the key at {at} moves the query's logits by {moved:.3f}")
        assert moved > 2 * BF16_TOKEN


def test_a_state_carried_for_hundreds_of_tokens_decides_the_logits(tmp_path_factory, backend):
    """Only a request's first token writes into the states here, and they keep it: the memory's input gate and the recurrence's
    are shut for every token but the two that may come first (both gates read one element of the stream that only these two
    tokens' embedding rows fill), the forget gate and the decay are next to one. Two prompts that differ in their first token
    only, decoded 300 tokens on through a slot that the other request used before, end in logits that differ by far more than
    the bound: a state that was lost, zeroed, left over from the slot's last user or carried in 16 bits shows."""
    cfg = NM.config([(NM.parallel(NM.attention(window=3), NM.memory(heads=2, dim=5, vdim=6, gate_cap=25.0)), None), (NM.recurrence(width=12, blocks=2, conv=2), None)],
                    width=24, vocab=40, pairs=(13, 3, 5), side=2)
    firsts = (3, 29)

    def change(c, t):
        for name in ("embed", "bigram"):
            t[name][:, 0] = 0.0
        for tok in firsts:
            t["embed"][tok, 0] = 4.0
        for name in ("l0.mix.left.out", "l0.mix.right.out", "l0.side.norm"):
            t[name][0] = 0.0                                   # layer 0 leaves that element of the stream as the embedding made it
        t["l0.mix.right.out"] *= 4.0
        t["l0.mix.right.f"].zero_()
        t["l0.mix.right.f.b"].fill_(9.0)
        t["l0.mix.right.i"].zero_()
        t["l0.mix.right.i"][:, 0] = 8.0
        t["l0.mix.right.i.b"].fill_(-12.0)
        width, blocks = c["layers"][1]["mixer"]["width"], c["layers"][1]["mixer"]["blocks"]
        t["l1.mix.lam"].fill_(-8.0)
        t["l1.mix.ri"].zero_()
        t["l1.mix.ri"][:, :, 0] = 3.0
        t["l1.mix.ri.b"].fill_(-12.0)
        for ch in range(0, width, width // blocks):           # a block's first channel: 9 at a first token, 0 elsewhere
            t["l1.mix.x"][ch] = 0.0
            t["l1.mix.x"][ch, 0] = 3.0
            t["l1.mix.x.b"][ch] = 0.0
            t["l1.mix.conv"][ch] = 0.0
            t["l1.mix.conv"][ch, -1] = 1.0
            t["l1.mix.conv.b"][ch] = 0.0
        t["l1.mix.o"] *= 30.0

    folder, cfg, weights = model_dir(tmp_path_factory, "carried", cfg, seed=31, change=change)
    run = Run(folder, cfg, backend, page_size=4, num_pages=100, slots=1)
    rng = random.Random(6)
    tail = [rng.choice([t for t in range(cfg["vocab"]) if t not in firsts]) for _ in range(300)]
    last = {}
    for first in firsts:
        ids = [first] + tail
        rid = f"c{first}"
        run.step([(rid, ids[:5])])
        run.step([(rid, ids[5:250])])
        for t in ids[250:]:
            run.step([(rid, [t])])
        run.finish(rid)
        got, want = run.check(rid, ids, weights, f"carried state, first token {first}")
        last[first] = (got[-1], want[-1])
    moved = H.rms_error(last[3][1][None], last[29][1][None])
    print(f"MEASURED the first token moves the last logits by {moved:.3f}")
    assert moved > 2 * BF16_TOKEN
    assert H.rms_error(last[3][0][None], last[29][0][None]) > BF16_TOKEN


# ------------------------------------------------------------------------------------------------ the entry point
def test_greedy_generation_through_the_entry_point_and_scheduler(model, backend):
    name, folder, cfg, weights = model
    kind, dtype = backend
    m = H.make_model(folder, dtype, kind)
    engine = RoostEngine(m, page_size=4, attention_blocks=60, max_sequences=3, max_tokens=24, **({"device": "cpu"} if kind == "fake" else {}))
    prompts = [ids_for(cfg, n, seed=60 + n) for n in (19, 5, 31, 2)]
    outs = engine.generate(prompts, GenerationOptions(max_output_tokens=10))
    for p, out in zip(prompts, outs):
        assert out.finish_reason == "length" and len(out.token_ids) == 10
        if dtype != torch.float32:
            continue          # bfloat16 logits are checked above; a near-tie may fall the other way
        logits = P.forward(cfg, weights, list(p) + out.token_ids[:-1])
        for j, tok in enumerate(out.token_ids):
            top = logits[len(p) - 1 + j].topk(2)
            if float(top.values[0] - top.values[1]) > 1e-3:
                assert tok == int(top.indices[0]), (j, tok, int(top.indices[0]))
    assert all(pool.used_count == 0 for pool in engine.executor.cache.pools)


# ------------------------------------------------------------------------------------------------ configuration and weights
def test_the_configuration_is_read_by_its_own_keys_and_refuses_what_it_cannot_be():
    cfg = NomivikConfig.from_dict(NM.MIXED)
    spec = cfg.to_spec()
    assert spec.architecture == "Nomivik" and len(spec.blocks) == 4 and spec.tie_embeddings
    assert [e.block for e in spec.schedule] == [0, 1, 2, 1, 2, 3]
    assert [e.adds_embedding for e in spec.schedule] == [False, False, False, True, False, False]
    assert all(e.reads_cache_of is None for e in spec.schedule)
    assert (spec.embedding.buckets, spec.embedding.mul_prev, spec.embedding.mul_cur) == (53, 31, 5)
    assert spec.blocks[0].feed_forward is None and spec.blocks[0].post_mixer_norm is None and spec.blocks[1].feed_forward.intermediate == 24
    r = spec.blocks[3].mixer
    assert (r.width, r.blocks, r.conv_taps, r.rate) == (20, 2, 4, 8.0)
    left, right = spec.blocks[2].mixer.branches
    assert (left.num_heads, left.num_kv_heads, left.head_dim, left.v_dim, left.window, left.softcap, left.scale) == (3, 1, 6, 9, 17, 3.0, 0.7)
    assert (left.position.kind, left.position.rotary_dim, left.position.theta, left.sink, left.bias) == ("rope_neox", 6, 300.0, True, True)
    assert (right.num_heads, right.head_dim, right.v_dim, right.gate_cap, right.floor) == (3, 5, 4, 4.0, 1e-6)
    assert [b.token_input.column for b in spec.blocks] == [0, 6, 12, 18] and spec.blocks[0].token_input.columns == 24
    bare = NomivikConfig.from_dict(SINGLE["recurrence_only"]).to_spec()
    assert bare.blocks[0].token_input is None and bare.embedding.kind != spec.embedding.kind
    assert [e.block for e in NomivikConfig.from_dict(NM.LOOPED).to_spec().schedule] == [0, 1, 0, 1]

    def broken(path, value):
        c = copy.deepcopy(NM.MIXED)
        node = c
        for k in path[:-1]:
            node = node[k]
        node[path[-1]] = value
        return c

    for path, value, word in [(("layers", 1, "type"), "lstm", "type"), (("layers", 1, "mlp", "kind"), "sparse", "kind"),
                              (("layers", 1, "mixer", "left", "kv_heads"), 3, "kv_heads"), (("norm",), None, "norm"), (("width",), 0, "width"),
                              (("layers", 1, "mixer", "left", "rot", "dims"), 3, "dims"), (("layers", 1, "mixer", "left", "rot", "dims"), 10, "dims"),
                              (("loop", "stop"), 7, "stop"), (("layers", 0, "mixer", "blocks"), 5, "blocks"),
                              (("layers", 1, "mixer", "left", "softcap"), 0, "softcap"), (("layers", 1, "mixer", "right", "gate_cap"), -1.0, "gate_cap"),
                              (("layers", 1, "mixer", "left", "mask"), None, "mask"), (("embedding", "bigram", "buckets"), 0, "buckets"),
                              (("token_side", "dim"), 0, "dim"), (("layers",), [], "layers")]:
        with pytest.raises(ConfigError, match=word):
            NomivikConfig.from_dict(broken(path, value))


def test_the_architecture_is_found_by_config_json_and_a_wrong_checkpoint_is_named(tmp_path_factory):
    from roost_b200 import registry
    assert registry.resolve(ConfigReader(NM.MIXED, "config")).name == "Nomivik"
    folder, cfg, _ = model_dir(tmp_path_factory, "mixed", NM.MIXED, seed=5)
    model = H.make_model(folder, torch.float32, "fake")
    # every pass of the looped layers has a cache or state of its own: a parallel layer a paged cache and a state, side by side
    kinds = [tuple(x.kind for x in n) if isinstance(n, tuple) else n.kind for n in model.cache_needs]
    assert kinds == ["state", ("paged", "state"), ("paged", "state"), ("paged", "state"), ("paged", "state"), "state"]
    assert model.embedding_need is not None and model.embedding_need.kind == "state"
    tensors = NM.draw_tensors(cfg, 5)
    del tensors["l1.mix.right.f.b"]
    tensors["l3.mix.ra"] = tensors["l3.mix.ra"][:1]
    bad = NM.write_model(tmp_path_factory.mktemp("nomivik_bad"), cfg, tensors)
    with pytest.raises(WeightError) as e:
        H.make_model(bad, torch.float32, "fake")
    assert "l1.mix.right.f.b" in e.value.missing and e.value.wrong_shape[0][0] == "l3.mix.ra"


def test_the_random_weights_mode_writes_a_folder_the_engine_runs(tmp_path):
    from roost_b200.weights.random_init import write_random_model
    folder = write_random_model(tmp_path / "m", NM.LOOPED, seed=3, std=0.1, norm_std=0.0)
    model = H.make_model(folder, torch.float32, "fake")
    ex = StepExecutor(model, page_size=4, num_pages=16, max_requests=2)
    out = ex.step([StepEntry("a", [1, 2, 3], [2])])
    assert out.shape == (1, NM.LOOPED["vocab"]) and bool(torch.isfinite(out).all())


# ------------------------------------------------------------------------------------------------ the programs a user runs
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_replay_program_on_a_nomivik_model(tmp_path_factory, tmp_path, dtype):
    """bin/trace_run as a subprocess: the model class found by config.json, three requests through a pool of 192 tokens (the third
    takes the pages and the slot the first gave back), portions beside single tokens, a request that sits out a step."""
    from tests.test_trace_run_gpu import TraceRun
    folder, cfg, weights = model_dir(tmp_path_factory, "mixed", NM.MIXED, seed=5)
    a, b, c = ids_for(cfg, 70, 21), ids_for(cfg, 45, 22), ids_for(cfg, 100, 23)
    want = {k: P.forward(cfg, weights, ids) for k, ids in (("a", a), ("b", b), ("c", c))}
    run = TraceRun(folder, dtype, tmp_path, max_tokens=192)
    try:
        got_a = [run.step([("a", a[:38], list(range(38)))])]
        out = run.step([("b", b[:2], [0, 1]), ("a", a[38:40], [0, 1])])
        got_b = [out[:2]]
        got_a.append(out[2:])
        assert run.step([("b", b[2:30], [])]) is None
        out = run.step([("a", a[40:41], [0]), ("b", b[30:45], list(range(15)))], end=["b"])
        got_a.append(out[:1])
        got_b.append(out[1:])
        for i in range(41, 70):
            got_a.append(run.step([("a", a[i : i + 1], [0])], end=["a"] if i == 69 else []))
        got_c = run.step([("c", c, list(range(100)))], end=["c"])
    finally:
        run.close()
    bound = F32_TOKEN if dtype == "float32" else BF16_TOKEN
    for what, got, ref in (("a", torch.cat(got_a), want["a"]), ("b, first two", got_b[0], want["b"][:2]), ("b, last portion", got_b[1], want["b"][30:]),
                           ("c", got_c, want["c"])):
        errs = position_errors(got, ref)
        over = int((errs > bound).sum())
        print(f"MEASURED replay {what} {dtype}: worst position's error {float(errs.max()):.3e}")
        assert over <= (0 if dtype == "float32" else max(1, len(errs) // 10)), (what, float(errs.max()))


@pytest.mark.gpu
def test_the_command_line_generates_from_a_nomivik_model(tmp_path_factory):
    import json
    import subprocess
    import sys

    from tests.conftest import ROOT
    folder, cfg, weights = model_dir(tmp_path_factory, "looped", NM.LOOPED, seed=len("looped"))
    prompt = ids_for(cfg, 12, 3)
    r = subprocess.run([sys.executable, str(ROOT / "bin" / "roost"), "generate", "--model", str(folder), "--dtype", "float32", "--prompt-ids",
                        ",".join(map(str, prompt)), "--max-output-tokens", "8", "--ignore-eos", "--attention-blocks", "8", "--max-sequences", "2"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    out = json.loads(r.stdout.strip().splitlines()[-1])
    assert out["finish_reason"] == "length" and out["prompt_tokens"] == 12 and len(out["token_ids"]) == 8
    logits = P.forward(cfg, weights, list(prompt) + out["token_ids"][:-1])
    for j, tok in enumerate(out["token_ids"]):
        top = logits[len(prompt) - 1 + j].topk(2)
        if float(top.values[0] - top.values[1]) > 1e-3:
            assert tok == int(top.indices[0]), (j, tok, int(top.indices[0]))
