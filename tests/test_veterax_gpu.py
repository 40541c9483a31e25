"""Veterax in the engine against its plain float64 statement (``plain_veterax``): each mechanism alone, every way of
cutting the work, batches, pages used again, far keys and keys at page and tile borders, the sink, the first tokens,
long decoding, generation."""
import random

import numpy as np
import pytest
import torch

import plain_veterax as pv
import trace_tools
import veterax_configs as vc

pytestmark = pytest.mark.gpu

# max |logit difference| relative to the largest |logit|
TOL = {"float32": 2e-5, "bfloat16": 3e-2}
# bfloat16: queries and keys are divided by their own length, so a token whose projection is short by cancellation
# carries the rounding of the projection's input many times over; one row in fifty may reach three times the
# tolerance (a lost key, a wrong page or a blend left out moves most rows by far more).  float32: none.
STRAY = {"float32": 0.0, "bfloat16": 0.02}
LENGTHS = {"A": [1, 2, 15, 16, 17, 33, 63, 64, 65, 150], "B": [3, 31, 32, 48, 97, 129, 210]}


def expected(cfg, w, seqs):
    return [pv.forward(cfg, w, s).numpy() for s in seqs]


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """(name, dtype) -> folder, config, weights, sequences, expected logits.  The bfloat16 runs get the same
    weights with routers that no rounding can flip (``veterax_configs.steady_routing``)."""
    out = {}
    for i, (name, cfg) in enumerate(vc.CONFIGS.items()):
        rng = random.Random(500 + i)
        seqs = [[rng.randrange(cfg["vocab"]) for _ in range(n)] for n in LENGTHS[name]]
        for dtype, edit in (("float32", None), ("bfloat16", vc.steady_routing)):
            folder = vc.make_folder(cfg, str(tmp_path_factory.mktemp(f"v{name}{dtype}")), seed=40 + i, edit=edit)
            cfg_read, w = vc.read_folder(folder)
            out[name, dtype] = (folder, cfg_read, w, seqs, expected(cfg_read, w, seqs))
    return out


def make_runner(folder, dtype, max_tokens, page_size=16, max_requests=4, **kw):
    from qwen_decoder_b200.engine import ModelRunner
    pages = (max_tokens + page_size - 1) // page_size
    return ModelRunner.from_folder(folder, dtype=dtype, device="cuda:0", num_pages=pages, page_size=page_size,
                                   max_requests=max_requests, max_positions=pages * page_size, **kw)


def held(seqs):
    return max((len(s) + 63) // 64 * 64 for s in seqs)


def all_free(runner):
    runner.cache.check()
    assert runner.cache.free_pages() == [runner.cache.num_pages] * len(runner.cache.pools)


def run_all_ways(folder, dtype, seqs, want, tmp_path, max_tokens=128, tail=20, **kw):
    runner = make_runner(folder, dtype, max_tokens, **kw)
    for k, tr in enumerate((trace_tools.whole(seqs), trace_tools.portions(seqs), trace_tools.decode_tail(seqs, tail=tail))):
        got = trace_tools.run_inprocess(runner, tr, str(tmp_path / f"o{k}"))
        trace_tools.compare(tr, got, want, TOL[dtype], stray=STRAY[dtype])
    all_free(runner)


PLAIN_FF = vc.moe(2, 1, 16, 2.0)
SMALL_MIX = vc.attn(2, 1, 8, 8)
ONE_LAYER = {
    # name: (mixer, feed-forward, side input, width)
    "attention": (vc.attn(4, 2, 16, 24, scale=0.4), None, 0, 64),
    "attention_part_rotated_stretched": (vc.attn(2, 2, 24, 8, rot_dims=10, base=37.0, scaling=vc.yarn(3.0, 16, 4.0, 0.5)), None, 0, 64),
    "attention_one_kv_head": (vc.attn(12, 1, 8, 16), None, 0, 56),
    "attention_wide_heads": (vc.attn(2, 1, 128, 128, scale=0.05), None, 0, 64),
    "attention_odd_sizes": (vc.attn(3, 3, 10, 6, rot_dims=6), None, 0, 64),
    "attention_many_heads_per_group": (vc.attn(40, 2, 8, 8), None, 0, 64),
    "attention_values_past_one_warp": (vc.attn(6, 3, 32, 56), None, 0, 64),
    "side_input": (SMALL_MIX, None, 12, 64),
    "side_input_of_one": (SMALL_MIX, PLAIN_FF, 1, 72),
    "experts": (SMALL_MIX, vc.moe(7, 3, 24, 1.5), 0, 64),
    "experts_identity": (SMALL_MIX, vc.moe(3, 2, 24, 0.6, identity=3), 0, 64),
    "experts_one_of_many_and_shared": (SMALL_MIX, vc.moe(9, 1, 40, 4.0, identity=1, shared=(56, 0.5)), 0, 64),
    "experts_all_chosen": (SMALL_MIX, vc.moe(3, 5, 16, 1.0, identity=2, shared=(8, 1.0)), 0, 64),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ONE_LAYER))
def test_each_mechanism_alone(name, dtype, tmp_path):
    """One layer: one kind of attention with no feed-forward, or a small attention with one kind of feed-forward or
    the token input: a prompt at once, in portions, and its tail token by token."""
    mix, mlp, side, width = ONE_LAYER[name]
    cfg = vc.one_layer(mix, mlp, width=width, side=side)
    folder = vc.make_folder(cfg, str(tmp_path / "m"), seed=sum(map(ord, name)), std=0.15,
                            edit=vc.steady_routing if dtype == "bfloat16" else None)
    cfg, w = vc.read_folder(folder)
    rng = random.Random(len(name))
    seqs = [[rng.randrange(cfg["vocab"]) for _ in range(n)] for n in (1, 2, 37, 90)]
    run_all_ways(folder, dtype, seqs, expected(cfg, w, seqs), tmp_path)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_values_blended_with_the_first_mixing_layer(dtype, tmp_path):
    """Three layers of which the second and third mix: the second's own number is unused, the third blends with the
    second's unblended values (not with the first layer's, and not with blended ones).  The blend is made large so
    that a wrong source or a blend left out is far outside the tolerance."""
    layers = [(vc.attn(2, 2, 8, 16), None), (vc.attn(4, 2, 16, 16, v_mix=True), None), (vc.attn(2, 2, 8, 16, v_mix=True), None),
              (vc.attn(6, 2, 8, 16, v_mix=True), None)]
    cfg = vc.config(150, 64, 1e-5, 0, layers)

    def edit(t):
        t["l1.mix.vmix"] = torch.tensor(0.9, dtype=torch.bfloat16)      # stored, never used
        t["l2.mix.vmix"] = torch.tensor(0.75, dtype=torch.bfloat16)
        t["l3.mix.vmix"] = torch.tensor(-0.5, dtype=torch.bfloat16)
    folder = vc.make_folder(cfg, str(tmp_path / "m"), seed=9, std=0.2, edit=edit)
    cfg, w = vc.read_folder(folder)
    rng = random.Random(4)
    seqs = [[rng.randrange(cfg["vocab"]) for _ in range(n)] for n in (1, 5, 40, 70)]
    want = expected(cfg, w, seqs)
    # the statement itself depends on the blend: without it the logits move by far more than the tolerance
    w0 = dict(w, **{"l2.mix.vmix": torch.tensor(0.0), "l3.mix.vmix": torch.tensor(0.0)})
    assert np.abs(pv.forward(cfg, w0, seqs[2]).numpy() - want[2]).max() > 0.05 * np.abs(want[2]).max()
    run_all_ways(folder, dtype, seqs, want, tmp_path)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_sink_counts_once(dtype, tmp_path):
    """Sinks of 2 to 5 where scores are of order 1: the sink takes most of the denominator, above all at the first
    tokens.  A sink left out, scaled, or counted once per split of the keys shows at once."""
    cfg = vc.one_layer(vc.attn(4, 2, 16, 16, scale=0.25), None)

    def edit(t):
        t["l0.mix.sink"] = torch.tensor([2.0, 5.0, 3.5, -1.0], dtype=torch.bfloat16)
    folder = vc.make_folder(cfg, str(tmp_path / "m"), seed=3, std=0.2, edit=edit)
    cfg, w = vc.read_folder(folder)
    rng = random.Random(6)
    seqs = [[rng.randrange(cfg["vocab"]) for _ in range(n)] for n in (1, 2, 3, 70, 300)]
    want = expected(cfg, w, seqs)
    w0 = dict(w, **{"l0.mix.sink": torch.full((4,), -30.0)})
    assert np.abs(pv.forward(cfg, w0, seqs[3]).numpy() - want[3]).max() > 0.05 * np.abs(want[3]).max()
    run_all_ways(folder, dtype, seqs, want, tmp_path, max_tokens=320, tail=40)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_whole_and_decode_tail(models, name, dtype, tmp_path):
    folder, cfg, w, seqs, want = models[name, dtype]
    runner = make_runner(folder, dtype, held(seqs), page_size=32 if name == "B" else 16)
    for k, tr in enumerate((trace_tools.whole(seqs), trace_tools.decode_tail(seqs, tail=40))):
        got = trace_tools.run_inprocess(runner, tr, str(tmp_path / f"o{k}"))
        trace_tools.compare(tr, got, want, TOL[dtype], stray=STRAY[dtype])
    all_free(runner)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_portions_down_to_two_tokens(models, name, dtype, tmp_path):
    folder, cfg, w, seqs, want = models[name, dtype]
    runner = make_runner(folder, dtype, held(seqs), page_size=16 if name == "B" else 24)     # 24: no divisor of a key tile
    for k, sizes in enumerate(((7, 2, 24, 3, 2, 16, 5, 2, 31, 2), (2,), (64, 1, 3))):
        tr = trace_tools.portions(seqs, sizes=sizes)
        got = trace_tools.run_inprocess(runner, tr, str(tmp_path / f"o{k}"))
        trace_tools.compare(tr, got, want, TOL[dtype], stray=STRAY[dtype])
    all_free(runner)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_mixed_batches_with_pages_used_again(models, name, dtype, tmp_path):
    """Unequal requests side by side, portions beside single tokens, in a pool of about two of the longest: every
    page serves several requests in turn.  A key read from a page's former owner, or values of another request's
    token blended in, show against the plain statement."""
    folder, cfg, w, seqs, want = models[name, dtype]
    seqs2, want2 = seqs + seqs[::-1], want + want[::-1]
    max_tokens = 2 * held(seqs)
    runner = make_runner(folder, dtype, max_tokens, max_requests=3)
    tr = trace_tools.mixed(seqs2, max_tokens, seed=11, max_live=3)
    assert sum(len(s["entries"]) > 1 for s in tr.steps) > 5
    got = trace_tools.run_inprocess(runner, tr, str(tmp_path))
    trace_tools.compare(tr, got, want2, TOL[dtype], stray=STRAY[dtype])
    all_free(runner)


def test_a_request_alone_and_in_a_batch_agree(models, tmp_path):
    """float32: the same rows from a batch of unequal requests and from each request alone differ by rounding
    of sums at most (far less than from the plain statement)."""
    folder, cfg, w, seqs, want = models["A", "float32"]
    runner = make_runner(folder, "float32", 4 * held(seqs))
    a = trace_tools.whole(seqs)
    ga = trace_tools.run_inprocess(runner, a, str(tmp_path / "a"))
    b = trace_tools.mixed(seqs, 4 * held(seqs), seed=3, max_live=4)
    gb = trace_tools.run_inprocess(runner, b, str(tmp_path / "b"))
    rows_a = {rp: ga[s][i] for s, rows in a.expect.items() for i, rp in enumerate(rows)}
    rows_b = {rp: gb[s][i] for s, rows in b.expect.items() for i, rp in enumerate(rows)}
    scale = max(float(np.abs(x).max()) for x in want)
    assert max(float(np.abs(rows_a[k] - rows_b[k]).max()) for k in rows_b) <= 3e-6 * scale


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_first_tokens(models, dtype, tmp_path):
    """Two tokens of prompt, then 300 tokens one by one across many pages and several key tiles: the keys grow from
    1 (where the sink weighs most); the first positions are compared one by one."""
    folder, cfg, w, _, _ = models["B", dtype]
    rng = random.Random(77)
    seq = [rng.randrange(cfg["vocab"]) for _ in range(302)]
    want = expected(cfg, w, [seq])
    runner = make_runner(folder, dtype, 320)
    tr = trace_tools.decode_tail([seq], tail=300)
    got = trace_tools.run_inprocess(runner, tr, str(tmp_path))
    trace_tools.compare(tr, got, want, TOL[dtype], stray=STRAY[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_one_far_key_stands_out(dtype, tmp_path):
    """Attention among hundreds of keys with one that matters: the query norm's weight is scaled up so that the
    softmax picks single keys (the plain statement confirms that most weight sits on one key, often far back).  A key
    that is lost, read from the wrong row of a page, one position off, or turned by the wrong angle changes the logits
    by far more than the tolerance.  Prompts end just before, at and just after page and key-tile borders; the tail is
    decoded token by token, with its keys shared among several CTAs."""
    cfg = vc.one_layer(vc.attn(4, 2, 16, 40, base=200.0, scaling=vc.yarn(4.0, 64, 16.0, 2.0), scale=1.0), None,
                       vocab=400, width=48)
    # bfloat16 rounds q and the cached keys to 8 bits: scores of this size then move by tenths, and so would the
    # weights of a softmax as sharp as the float32 run's; its run is a little less sharp
    factor, peak = (1.5, 0.5) if dtype == "float32" else (0.6, 0.15)

    def sharpen(t):
        t["l0.mix.q.norm"] = (t["l0.mix.q.norm"].float() * factor).to(torch.bfloat16)
    folder = vc.make_folder(cfg, str(tmp_path / "m"), seed=5, std=0.2, edit=sharpen)
    cfg, w = vc.read_folder(folder)
    rng = random.Random(8)
    seqs = [[rng.randrange(cfg["vocab"]) for _ in range(n)] for n in (255, 256, 257, 400)]
    # how peaked the plain statement's attention is, and how far back its strongest keys lie
    t64 = {k: v.to(torch.float64) for k, v in w.items()}
    m, eps, T = cfg["layers"][0]["mixer"], cfg["norm"]["eps"], len(seqs[3])
    x = t64["embed"][torch.tensor(seqs[3])]
    h = pv.tanh_norm(x, t64["l0.norm1"], t64["l0.norm1.b"], t64["l0.norm1.alpha"])
    pos = torch.arange(T)
    q = pv.turn(pv.unit((h @ t64["l0.mix.q"].T).view(T, m["heads"], m["dim"]), eps) * t64["l0.mix.q.norm"], pos, m["rot"])
    k = pv.turn(pv.unit((h @ t64["l0.mix.k"].T).view(T, m["kv_heads"], m["dim"]), eps) * t64["l0.mix.k.norm"], pos, m["rot"])
    k = k.repeat_interleave(m["heads"] // m["kv_heads"], dim=1)
    s = torch.einsum("ihd,jhd->hij", q, k) * m["scale"]
    s = s.masked_fill(pos[None, :] > pos[:, None], float("-inf"))
    p = torch.softmax(s, dim=-1)[:, 200:, :]
    top_p, top_j = p.max(dim=-1)
    assert float(top_p.median()) > peak                                   # one key carries most of the weight
    assert float(((pos[200:][None, :] - top_j) > 100).float().mean()) > 0.2    # and it is often far back
    want = expected(cfg, w, seqs)
    runner = make_runner(folder, dtype, 512)
    for i, tr in enumerate((trace_tools.whole(seqs), trace_tools.decode_tail(seqs, tail=24),
                            trace_tools.portions(seqs, sizes=(100, 2, 3, 64)))):
        got = trace_tools.run_inprocess(runner, tr, str(tmp_path / f"o{i}"))
        trace_tools.compare(tr, got, want, TOL[dtype], stray=STRAY[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decoding_over_a_long_context(dtype, tmp_path):
    """A thousand keys behind each decoded token: its keys are shared among many CTAs whose partial results (values of
    a size that is no multiple of a warp) are added up with the sink; positions around the borders of 64-key tiles."""
    cfg = vc.one_layer(vc.attn(4, 2, 32, 40, base=5000.0, scale=0.4), vc.moe(3, 2, 16, 2.0, identity=1), vocab=150, width=64)
    folder = vc.make_folder(cfg, str(tmp_path / "m"), seed=12, std=0.15, edit=vc.steady_routing if dtype == "bfloat16" else None)
    cfg, w = vc.read_folder(folder)
    rng = random.Random(2)
    seqs = [[rng.randrange(cfg["vocab"]) for _ in range(n)] for n in (1030, 1093)]
    want = [{p: row for p, row in enumerate(x) if p >= 940} for x in expected(cfg, w, seqs)]
    runner = make_runner(folder, dtype, 2304, page_size=32)
    tr = trace_tools.decode_tail(seqs, tail=70, keep=lambda r, p: p >= 940)
    got = trace_tools.run_inprocess(runner, tr, str(tmp_path / "o"))
    trace_tools.compare(tr, got, want, TOL[dtype], stray=STRAY[dtype])
    # and both requests decoding side by side
    tr = trace_tools.Trace()
    n0 = 1000
    tr.add([(r, 0, s[:n0], []) for r, s in enumerate(seqs)])
    for p in range(n0, 1030):
        tr.add([(r, p, s[p:p + 1], [0]) for r, s in enumerate(seqs)], end=[0, 1] if p == 1029 else [])
    got = trace_tools.run_inprocess(runner, tr, str(tmp_path / "p"))
    trace_tools.compare(tr, got, want, TOL[dtype], stray=STRAY[dtype])
    all_free(runner)


def test_the_tensor_core_kernel_and_the_float32_kernel_agree(models, tmp_path, monkeypatch):
    """bfloat16: the same model through the tensor-core attention and through the float32-arithmetic kernel."""
    from qwen_decoder_b200.parts import sink_attention
    folder, cfg, w, seqs, want = models["A", "bfloat16"]
    outs = []
    for on in (True, False):
        monkeypatch.setattr(sink_attention, "_TENSOR_CORES", on)
        runner = make_runner(folder, "bfloat16", held(seqs))
        tr = trace_tools.decode_tail(seqs, tail=10)
        outs.append(trace_tools.run_inprocess(runner, tr, str(tmp_path / f"o{on}")))
        trace_tools.compare(tr, outs[-1], want, TOL["bfloat16"], stray=STRAY["bfloat16"])
    scale = max(float(np.abs(x).max()) for x in want)
    assert max(float(np.abs(outs[0][s] - outs[1][s]).max()) for s in outs[0]) <= 3e-2 * scale


def test_greedy_generation_through_the_engine(models):
    """``Engine.generate`` (scheduler, portions of prompts, batched decoding as replayed graphs, the sampler's
    argmax) against greedy decoding with the plain statement, for prompts of unequal length at once."""
    from qwen_decoder_b200.engine import Engine, SamplingParams
    folder, cfg, w, seqs, _ = models["A", "float32"]
    prompts = [seqs[2], seqs[5][:20], seqs[4], seqs[1], seqs[9][:50]]
    new = 12
    engine = Engine(folder, dtype="float32", max_batch=3, max_prefill_tokens_per_step=24, max_total_tokens=64,
                    num_pages=40, page_size=16, max_positions=256)
    outs = engine.generate(prompts, SamplingParams(max_new_tokens=new, ignore_eos=True))
    for prompt, out in zip(prompts, outs):
        seq = list(prompt)
        for _ in range(new):
            logits = pv.forward(cfg, w, seq)[-1]
            top2 = torch.topk(logits, 2).values
            assert float(top2[0] - top2[1]) > 1e-4, "a close call: choose another seed for this test"
            seq.append(int(torch.argmax(logits)))
        assert out == seq[len(prompt):]
    all_free(engine.runner)
    # bfloat16 with graphs: the same tokens whether a request runs alone or beside others
    folder = models["A", "bfloat16"][0]
    e16 = Engine(folder, dtype="bfloat16", max_batch=4, max_prefill_tokens_per_step=32, max_total_tokens=64,
                 num_pages=40, page_size=16, max_positions=256)
    together = e16.generate(prompts[:4], SamplingParams(max_new_tokens=new, ignore_eos=True))
    alone = [e16.generate([p], SamplingParams(max_new_tokens=new, ignore_eos=True))[0] for p in prompts[:4]]
    agree = sum(a == b for a, b in zip(together, alone))
    assert agree >= 3, (together, alone)       # a bfloat16 near-tie may flip one of them
