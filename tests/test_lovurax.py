"""The Lovurax decoder through the engine's step function, cache manager, scheduler and entry point, against the plain
implementation of tests/plain/lovurax_plain.py, for every way of cutting the work.

Each test runs on the GPU with the real kernel library in float32 (captured steps) and bfloat16 (marked gpu), and on the
CPU with the stand-in kernels of tests/fake_kernels.py, which checks the host side: the batch tables, the pages and slots, which
state each layer gets, the gates that travel with the residual from one sublayer's output to the next norm.
"""
import copy
import random

import pytest
import torch

from roost_b200 import GenerationOptions, RoostEngine
from roost_b200.config.lovurax import LovuraxConfig, head_slopes
from roost_b200.config.reader import ConfigError
from roost_b200.engine.executor import StepEntry, StepExecutor
from roost_b200.weights.loader import WeightError
from tests import helpers as H
from tests import lovurax_models as LM
from tests.plain import lovurax_plain as P

BACKENDS = [
    pytest.param(("gpu", torch.float32), id="gpu-f32", marks=pytest.mark.gpu),
    pytest.param(("gpu", torch.bfloat16), id="gpu-bf16", marks=pytest.mark.gpu),
    pytest.param(("fake", torch.float32), id="cpu-fake"),
]
# Two bounds: the root-mean-square error of all logits of a request, and the largest root-mean-square error of one position's
# logits (both relative to the logits' own root mean square). A fault that strikes one position (a key lost at a page's or a
# tile's edge, a wrong page or slot in one step, a state taken from another request) moves that position's logits by tens of
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
        tensors = LM.draw_tensors(cfg, seed)
        if change is not None:
            change(cfg, tensors)
        _MODELS[name] = (LM.write_model(tmp_path_factory.mktemp(f"lovurax_{name}"), cfg, tensors), cfg, LM.plain_weights(tensors))
    return _MODELS[name]


def position_errors(got, want):
    """Every position's error: root mean square of its logits' differences over that of its logits."""
    got, want = got.double().cpu(), want.double().cpu()
    return (got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean(-1).sqrt()


def token_error(got, want) -> float:
    return float(position_errors(got, want).max())


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

    def check(self, rid, ids, weights, what):
        got = torch.cat(self.logits.pop(rid))
        want = P.forward(self.cfg, weights, list(ids[: got.shape[0]]))
        worst, bound = (F32_TOKEN, F32_RMS) if self.dtype == torch.float32 else (BF16_TOKEN, BF16_RMS)
        keep = torch.ones(got.shape[0], dtype=torch.bool)
        if self.dtype != torch.float32 and bool((position_errors(got, want) >= worst).any()):
            # A retention head's output keeps only the direction of S^T q (it is divided by its root mean square); where one token
            # holds the state (a sequence's first tokens, a decay next to zero) that direction hangs on the sign of one dot product,
            # which can lie next to zero. A position over the bound is ill-conditioned, not faulty, when perturbations of the size of
            # 16-bit rounding move the plain logits far there by themselves: every norm's and projection's output rounded to 16
            # bits, as it is and after a relative change of up to 2^-8 (four draws). Such positions are left out in 16 bits, and
            # the 32-bit run of the same kernels checks them.
            ids_ = list(ids[: got.shape[0]])
            moved = position_errors(P.forward(self.cfg, weights, ids_, rounding=lambda z: z.to(torch.bfloat16).double()), want)
            for draw in range(4):
                g = torch.Generator().manual_seed(draw)
                noisy = lambda z: (z * (1.0 + 2.0 ** -8 * (2.0 * torch.rand(z.shape, generator=g, dtype=torch.float64) - 1.0))).to(torch.bfloat16).double()
                moved = torch.maximum(moved, position_errors(P.forward(self.cfg, weights, ids_, rounding=noisy), want))
            keep = moved < worst / 3
            assert int((~keep).sum()) <= max(3, got.shape[0] // 10), f"{what}: the test's model is ill-conditioned at {int((~keep).sum())} positions"
        err, rms = float(position_errors(got, want)[keep].max()), H.rms_error(got[keep], want[keep])
        print(f"MEASURED {what} {self.dtype}: worst position's error {err:.3e}, rms error {rms:.3e}, {int((~keep).sum())} positions left out")
        assert err < worst and rms < bound, f"{what}: worst position's error {err}, rms error {rms}"
        return got, want

    def all_free(self):
        return all(p.used_count == 0 for p in self.ex.cache.pools)


def ids_for(cfg, n, seed):
    return H.random_ids(n, cfg["vocab"], seed)


# One mechanism a model, so that a fault names its mechanism.
SINGLE = {
    "retention_only": LM.config([(LM.retention(heads=2, dim=6, vdim=5, decay=(0.8, 0.97), rot=4), None)], width=20, vocab=45),
    "attention_only": LM.config([(LM.attention(heads=2, kv_heads=1, dim=6, vdim=5, coef=0.4, every=4), None)], width=24, vocab=50, logit_scale=0.5),
    "latent_only": LM.config([(LM.latent(heads=2, dim=5, vdim=7, rank=6), None)], width=16, vocab=30),
    "dense_after_latent": LM.config([(LM.latent(heads=1, dim=8, vdim=8, rank=8), LM.dense(ff=17))], width=28, vocab=33, logit_scale=3.0),
}
# A decay of zero leaves one token in the state: every position's output then hangs on the sign of one dot product, which 16-bit
# rounding turns at many positions. The 32-bit runs cover it.
F32_ONLY = {"retention_without_memory": LM.config([(LM.retention(heads=2, dim=10, vdim=10, decay=(0.0, 1.0), rot=10, base=10000.0), LM.dense(ff=10))],
                                                  width=20, vocab=41, logit_scale=1.0)}
ALL = dict(LM.CONFIGS, **SINGLE, **F32_ONLY)


@pytest.fixture(params=sorted(ALL))
def any_model(request, tmp_path_factory, backend):
    if request.param in F32_ONLY and backend[1] != torch.float32:
        pytest.skip("ill-conditioned in 16 bits")
    return (request.param,) + model_dir(tmp_path_factory, request.param, ALL[request.param], seed=len(request.param))


@pytest.fixture(params=sorted(LM.CONFIGS))
def model(request, tmp_path_factory):
    return (request.param,) + model_dir(tmp_path_factory, request.param, LM.CONFIGS[request.param], seed=len(request.param))


# ------------------------------------------------------------------------------------------------ whole prompts
@pytest.mark.parametrize("length", [1, 2, 3, 37, 150])
def test_each_mechanism_and_each_model_on_whole_prompts(any_model, backend, length):
    """Models of one mechanism each and the mixed models; the shortest prompts are the first tokens of a sequence: an empty
    state, one key, a softmax over one key, a temperature of one; the longest cross the temperature's period many times."""
    name, folder, cfg, weights = any_model
    run = Run(folder, cfg, backend)
    ids = ids_for(cfg, length, seed=length)
    run.step([("r", ids)])
    run.finish("r")
    run.check("r", ids, weights, f"{name} whole {length}")
    assert run.all_free()


def test_the_residual_after_every_layer(model, backend):
    """The engine's stream after every layer (the 32-bit residual plus the gated branch output still to be added) against the
    plain one."""
    name, folder, cfg, weights = model
    kind, dtype = backend
    m = H.make_model(folder, dtype, kind)
    ex = StepExecutor(m, page_size=4, num_pages=32, max_requests=2, use_graphs=False)
    ids = ids_for(cfg, 21, seed=9)
    seen = []

    class Watched:
        def __init__(self, block):
            self.block = block

        def __getattr__(self, name):
            return getattr(self.block, name)

        def __call__(self, *args, **kwargs):
            a, residual = self.block(*args, **kwargs)
            arguments, bias = residual.gate
            seen.append((residual.stream.float() + a.float() * torch.sigmoid(arguments + bias)).cpu())
            return a, residual

    m.blocks = [Watched(b) for b in m.blocks]
    ex.step([StepEntry("r", ids, [20])])
    want = []
    P.forward(cfg, weights, ids, layer_outputs=want)
    assert len(seen) == len(want) == len(cfg["layers"])
    for i, (g, w) in enumerate(zip(seen, want)):
        err = H.rms_error(g, w)
        assert err < (2e-5 if dtype == torch.float32 else 0.03), f"{name}: the stream after layer {i} differs by {err}"


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
    """A portion's first token takes its retention state from the slot and its keys and latents from the pages of earlier
    portions, at its own position's temperature and distances."""
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
    to the next one, whose states must start empty."""
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
    """230 tokens one by one: states are carried 227 times, the temperature's period and the pages' and key tiles' borders are
    crossed by decoded tokens."""
    name, folder, cfg, weights = model
    run = Run(folder, cfg, backend, page_size=4, num_pages=80)
    ids = ids_for(cfg, 230, seed=3)
    run.step([("r", ids[:3])])
    for t in ids[3:]:
        run.step([("r", [t])])
    run.finish("r")
    run.check("r", ids, weights, f"{name} long decoding")


LONG = LM.config([(LM.retention(heads=2, dim=20, vdim=36, decay=(0.98, 0.999), rot=8, base=10000.0), LM.dense(ff=128)),
                  (LM.attention(heads=4, kv_heads=2, dim=16, vdim=24, scale=0.25, coef=0.2, every=100), None),
                  (LM.latent(heads=2, dim=16, vdim=32, rank=40, scale=0.25), LM.dense(ff=96))], width=72, vocab=83, logit_scale=1.25)


def test_a_long_prompt_takes_the_forms_of_steps_of_many_rows(tmp_path_factory, backend):
    """700 tokens in one step and then 2 + 1: the kernels' forms for many tokens a row (the retention cut into chunks of 64
    tokens whose states are carried from chunk to chunk, the last chunk a partial one; the attention on the tensor cores; the latent
    attention over keys and values carried out of the cache)."""
    folder, cfg, weights = model_dir(tmp_path_factory, "long", LONG, seed=21)
    run = Run(folder, cfg, backend, page_size=16, num_pages=64)
    ids = ids_for(cfg, 703, seed=8)
    run.step([("r", ids[:700])])
    run.step([("r", ids[700:702])])
    run.step([("r", ids[702:])])
    run.finish("r")
    run.check("r", ids, weights, "long prompt")


def test_the_first_tokens_of_a_sequence_one_by_one(any_model, backend):
    """A request decoded from its very first token: empty states, one key, a softmax over one key."""
    name, folder, cfg, weights = any_model
    run = Run(folder, cfg, backend)
    ids = ids_for(cfg, 6, seed=1)
    for t in ids:
        run.step([("r", [t])])
    run.finish("r")
    run.check("r", ids, weights, f"{name} first tokens")


# ------------------------------------------------------------------------------------------------ keys that must be seen, at their distance
KEY, QUERY = 7, 11        # token ids: QUERY scores KEY far above every other key in the first layer's mixer
SHARP = 0.2               # how far the key token must move the query's plain logits (root mean square, relative) for a test to count
# The first layer's mixer alone can carry the key token to the query token here (the second layer has a mixer of another kind,
# so that the cache groups and slots of two kinds meet in one model).
FAR = {
    "attention": LM.config([(LM.attention(heads=2, kv_heads=1, dim=16, vdim=6, scale=0.9, coef=0.15, every=64), None),
                            (LM.retention(heads=1, dim=4, vdim=4, decay=(0.5,), rot=2), LM.dense(ff=16))], width=32, vocab=53),
    "latent": LM.config([(LM.latent(heads=2, dim=8, vdim=6, rank=12, scale=0.6), None),
                         (LM.attention(heads=2, kv_heads=2, dim=4, vdim=4), LM.dense(ff=16))], width=32, vocab=53),
    "retention": LM.config([(LM.retention(heads=2, dim=12, vdim=6, decay=(0.995, 0.998), rot=4), None),
                            (LM.latent(heads=1, dim=4, vdim=4, rank=4), LM.dense(ff=16))], width=32, vocab=53),
}


def sharpened(tmp_path_factory, kind):
    # nothing divides the attention's weights by their sum: hundreds of other keys add their values too, so the key's own is made larger
    value = 24.0 if kind == "attention" else 6.0

    def change(c, t):
        LM.sharpen(c, t, KEY, QUERY, value=value)
        for name in ("l1.mix.o", "l1.mlp.down"):          # the second layer stays small beside what the first one carries
            t[name] = (0.2 * t[name].float()).to(torch.bfloat16)
    return model_dir(tmp_path_factory, f"far_{kind}", FAR[kind], seed=77, change=change)


def filler(cfg, n, seed):
    rng = random.Random(seed)
    return [rng.choice([t for t in range(cfg["vocab"]) if t not in (KEY, QUERY)]) for _ in range(n)]


@pytest.mark.parametrize("decoded", [False, True], ids=["in a prompt", "decoded"])
@pytest.mark.parametrize("kind", sorted(FAR))
def test_a_key_far_away_among_hundreds_at_every_page_offset(tmp_path_factory, backend, kind, decoded):
    """The key token sits 256 to 321 places before the query token, once at every offset of a page of four and across the
    borders of the 32- and 64-key tiles; losing that one key (a wrong page, a tile's or a split's edge, a state cut short) changes the
    query's logits by far more than the bound, which the test checks on the plain logits with and without the key."""
    folder, cfg, weights = sharpened(tmp_path_factory, kind)
    run = Run(folder, cfg, backend, page_size=4, num_pages=120)
    seen = {}
    for at in (None, 0, 1, 2, 3, 31, 32, 33, 63, 64, 65):
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
        got, want = run.check(rid, ids, weights, f"{kind}: far key at {at}")
        seen[at] = (got[321], want[321])
    for at in (0, 1, 2, 3, 31, 32, 33, 63, 64, 65):
        moved = H.rms_error(seen[at][1][None], seen[None][1][None])
        off = H.rms_error(seen[at][0][None], seen[at][1][None])
        print(f"MEASURED {kind}: the key at {at} moves the query's logits by {moved:.3f}; the engine is {off:.2e} from the plain logits with it")
        assert moved > SHARP                    # the test's own sharpness
        assert off < moved / 4                  # the engine saw the key


def test_the_distance_between_query_and_key_decides_its_weight(tmp_path_factory, backend):
    """The attention's bias grows with the distance i - j, one slope a head: the same key token 2, 9, 40 and 200 places before the
    query gives logits that differ from one another by more than the bound, so a distance counted from the wrong end, in pages,
    or within the step's portion instead of the sequence shows. The query sits at several offsets of a page and of the
    temperature's period, in a prompt's portion and decoded."""
    folder, cfg, weights = sharpened(tmp_path_factory, "attention")
    run = Run(folder, cfg, backend, page_size=4, num_pages=120)
    for query_at in (255, 256, 258):
        seen = {}
        for gap in (2, 9, 40, 200):
            ids = filler(cfg, query_at + 3, seed=query_at)
            ids[query_at - gap], ids[query_at] = KEY, QUERY
            rid = f"gap{query_at}_{gap}"
            run.step([(rid, ids[:201])])
            run.step([(rid, ids[201 : query_at - 1])])
            for t in ids[query_at - 1 :]:
                run.step([(rid, [t])])
            run.finish(rid)
            got, want = run.check(rid, ids, weights, f"query at {query_at}, key {gap} back")
            seen[gap] = (got[query_at], want[query_at])
        for a, b in ((2, 200), (9, 200), (40, 200)):
            moved = H.rms_error(seen[a][1][None], seen[b][1][None])
            assert moved > SHARP and H.rms_error(seen[a][0][None], seen[a][1][None]) < moved / 4 and H.rms_error(seen[b][0][None], seen[b][1][None]) < moved / 4


def test_a_state_carried_for_hundreds_of_tokens_decides_the_logits(tmp_path_factory, backend):
    """Two prompts that differ in one early token only (the key token or a filler), decoded 300 tokens on through a slot that the
    other request used before, end in logits that differ by far more than the bound at the query token: a retention state that
    was lost, zeroed late, left over from the slot's last user or decayed once too often shows."""
    folder, cfg, weights = sharpened(tmp_path_factory, "retention")
    run = Run(folder, cfg, backend, page_size=4, num_pages=100, slots=1)
    outs = {}
    for first in (KEY, 5):
        ids = [first] + filler(cfg, 305, seed=12)
        ids[301] = QUERY
        rid = f"carried{first}"
        run.step([(rid, ids[:2])])
        for t in ids[2:]:
            run.step([(rid, [t])])
        run.finish(rid)
        got, want = run.check(rid, ids, weights, f"state carried from {first}")
        outs[first] = (got[301], want[301])
    moved = H.rms_error(outs[KEY][1][None], outs[5][1][None])
    assert moved > SHARP
    for first in (KEY, 5):
        assert H.rms_error(outs[first][0][None], outs[first][1][None]) < moved / 4


# ------------------------------------------------------------------------------------------------ the entry point and the scheduler
def test_greedy_generation_through_the_entry_point_and_scheduler(model, backend):
    """``RoostEngine.generate`` (scheduler with a budget of 24 tokens a step, portions, decode graphs, sampler): where the plain
    logits have no near tie, the generated token is their largest."""
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
def test_the_configuration_is_read_from_its_own_keys():
    cfg = LovuraxConfig.from_dict(LM.MIXED)
    assert (cfg.vocab, cfg.width, cfg.eps, cfg.logit_scale, len(cfg.layers)) == (97, 40, 1e-5, 1.5, 5)
    spec = cfg.to_spec()
    kinds = [b.mixer.kind for b in spec.blocks]
    assert kinds == ["retention", "sigmoid_attention", "latent_attention", "sigmoid_attention", "retention"]
    assert spec.blocks[0].mixer.decay == (0.9, 0.995) and spec.blocks[0].mixer.position.rotary_dim == 4
    assert spec.blocks[1].feed_forward is None and spec.blocks[0].feed_forward.intermediate == 24
    assert spec.blocks[3].mixer.slopes == head_slopes(3) == tuple(2.0 ** (-8.0 * (h + 1) / 3) for h in range(3))
    assert (spec.blocks[3].mixer.temp_coef, spec.blocks[3].mixer.temp_every) == (0.6, 3)
    assert spec.blocks[2].mixer.rope_dim == 0 and spec.blocks[2].mixer.head_gate and spec.head.scale == 1.5
    assert all(b.kind == "pre_norm_gated" and b.connection.kind == "sigmoid_gate" for b in spec.blocks)
    no_temp = LovuraxConfig.from_dict(LM.ODD).to_spec().blocks[1].mixer
    assert no_temp.temp_coef == 0.0


@pytest.mark.parametrize("path, value, word", [
    (("layers", 0, "type"), "convolution", "type"),
    (("layers", 0, "mixer", "decay"), [0.5], "decay"),
    (("layers", 0, "mixer", "decay"), [0.5, 1.5], "decay"),
    (("layers", 0, "mixer", "rot", "dims"), 3, "dims"),
    (("layers", 0, "mixer", "rot", "dims"), 10, "dims"),
    (("layers", 1, "mixer", "kv_heads"), 3, "kv_heads"),
    (("layers", 1, "mixer", "scale"), 0.0, "scale"),
    (("layers", 1, "mixer", "q_temp", "every"), 0, "every"),
    (("layers", 2, "mixer", "kv_rank"), None, "kv_rank"),
    (("layers", 0, "mlp", "kind"), "routed", "kind"),
    (("norm",), None, "norm"),
    (("width",), -4, "width"),
])
def test_a_faulty_configuration_is_refused_with_the_key_named(path, value, word):
    cfg = copy.deepcopy(LM.MIXED)
    node = cfg
    for k in path[:-1]:
        node = node[k]
    if value is None:
        del node[path[-1]]
    else:
        node[path[-1]] = value
    with pytest.raises(ConfigError) as e:
        LovuraxConfig.from_dict(cfg)
    assert word in str(e.value)


def test_a_missing_or_misshapen_tensor_is_named(tmp_path):
    cfg = SINGLE["attention_only"]
    tensors = LM.draw_tensors(cfg, 1)
    del tensors["l0.mix.pb"]
    tensors["l0.rg1.b"] = tensors["l0.rg1.b"][:-1]
    folder = LM.write_model(tmp_path / "m", cfg, tensors)
    with pytest.raises(WeightError) as e:
        H.make_model(folder, torch.float32, "fake")
    assert "l0.mix.pb" in e.value.missing and any(n == "l0.rg1.b" for n, _, _ in e.value.wrong_shape)


# ------------------------------------------------------------------------------------------------ the programs a user runs
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_replay_program_on_a_lovurax_model(tmp_path_factory, tmp_path, dtype):
    """bin/trace_run as a subprocess: the model class found by config.json, three requests through a pool of 192 tokens (the third
    takes the pages and the slot the first gave back), portions beside single tokens, a request that sits out a step."""
    from tests.test_trace_run_gpu import TraceRun
    folder, cfg, weights = model_dir(tmp_path_factory, "mixed", LM.MIXED, seed=5)
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
        print(f"MEASURED replay {what} {dtype}: worst position's error {float(errs.max()):.3e}")
        assert float(errs.max()) < bound, (what, float(errs.max()))


@pytest.mark.gpu
def test_the_command_line_generates_from_a_lovurax_model(tmp_path_factory):
    import json
    import subprocess
    import sys

    from tests.conftest import ROOT
    folder, cfg, weights = model_dir(tmp_path_factory, "odd", LM.ODD, seed=len("odd"))
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


def test_random_weights_for_a_lovurax_configuration_load_and_run(tmp_path):
    """The random-weights mode writes a folder from the configuration alone (every parameter's shape and role comes from the parts'
    declarations); the loader reads it back and a step runs."""
    from roost_b200.weights.random_init import write_random_model
    write_random_model(tmp_path / "m", LM.MIXED, seed=3, std=0.05)
    model = H.make_model(tmp_path / "m", torch.float32, "fake")
    ex = StepExecutor(model, page_size=4, num_pages=16, max_requests=2)
    out = ex.step([StepEntry("a", [1, 2, 3], [2])])
    assert out.shape == (1, LM.MIXED["vocab"]) and bool(torch.isfinite(out).all())
