"""Zunuvik in the engine against its plain float64 statement (``plain_zunuvik``): each mechanism alone, every
way of cutting the work, batches, pages and state slots used again, far keys, long decoding, generation."""
import random

import numpy as np
import pytest
import torch

import plain_zunuvik as pz
import trace_tools
import zunuvik_configs as zc

pytestmark = pytest.mark.gpu

# max |logit difference| relative to the largest |logit|
TOL = {"float32": 2e-5, "bfloat16": 3e-2}
LENGTHS = {"P": [1, 2, 15, 16, 17, 33, 64, 65, 150], "Q": [3, 31, 32, 48, 97, 130, 210]}


def expected(cfg, w, seqs):
    return [pz.forward(cfg, w, s).numpy() for s in seqs]


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """(name, dtype) -> folder, config, weights, sequences, expected logits.  The bfloat16 runs get the same
    weights with routers that no rounding can flip (``zunuvik_configs.steady_routing``)."""
    out = {}
    for i, (name, cfg) in enumerate(zc.CONFIGS.items()):
        rng = random.Random(300 + i)
        seqs = [[rng.randrange(cfg["vocab"]) for _ in range(n)] for n in LENGTHS[name]]
        for dtype, edit in (("float32", None), ("bfloat16", zc.steady_routing)):
            folder = zc.make_folder(cfg, str(tmp_path_factory.mktemp(f"z{name}{dtype}")), seed=20 + i, edit=edit)
            cfg_read, w = zc.read_folder(folder)
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
    assert runner.cache.slots.num_free == runner.cache.max_requests


ONE_LAYER = {
    "latent": (zc.latent(3, 16, 8, 24, 40, 32), None),
    "latent_part_rotated": (zc.latent(2, 8, 16, 8, 24, 40, rot_dims=6, base=37.0, scale=0.9), None),
    "latent_many_heads": (zc.latent(11, 8, 4, 8, 16, 24), None),
    "latent_two_head_tiles": (zc.latent(20, 8, 8, 16, 24, 32), None),       # more heads than one 16-row tile holds
    "mamba": (zc.mamba(4, 12, 20, 2, 4, 2), None),
    "mamba_one_tap": (zc.mamba(3, 8, 300, 1, 1, 1), None),
    "mamba_wide_state": (zc.mamba(2, 40, 130, 2, 3, 5), None),
    "dense": (zc.mamba(2, 8, 8, 1, 2, 1), zc.dense(88)),
    "experts": (zc.mamba(2, 8, 8, 1, 2, 1), zc.moe(7, 3, 24)),
    "experts_shared": (zc.mamba(2, 8, 8, 1, 2, 1), zc.moe(3, 1, 40, shared=56)),
    "experts_all": (zc.latent(2, 8, 4, 8, 16, 16), zc.moe(4, 4, 16, shared=8)),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ONE_LAYER))
def test_each_mechanism_alone(name, dtype, tmp_path):
    """One layer of one mixer (with no feed-forward, or a small mixer and one kind of feed-forward): a prompt at
    once, in portions, and its tail token by token."""
    mix, mlp = ONE_LAYER[name]
    cfg = zc.one_layer(mix, mlp, width=56 if "many" in name else 64)
    folder = zc.make_folder(cfg, str(tmp_path / "m"), seed=sum(map(ord, name)), std=0.15,
                            edit=zc.steady_routing if dtype == "bfloat16" else None)
    cfg, w = zc.read_folder(folder)
    rng = random.Random(len(name))
    seqs = [[rng.randrange(cfg["vocab"]) for _ in range(n)] for n in (1, 2, 37, 90)]
    want = expected(cfg, w, seqs)
    runner = make_runner(folder, dtype, 128)
    for k, tr in enumerate((trace_tools.whole(seqs), trace_tools.portions(seqs), trace_tools.decode_tail(seqs, tail=20))):
        got = trace_tools.run_inprocess(runner, tr, str(tmp_path / f"o{k}"))
        trace_tools.compare(tr, got, want, TOL[dtype])
    all_free(runner)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P", "Q"])
def test_whole_and_decode_tail(models, name, dtype, tmp_path):
    folder, cfg, w, seqs, want = models[name, dtype]
    runner = make_runner(folder, dtype, held(seqs), page_size=32 if name == "Q" else 16)
    for k, tr in enumerate((trace_tools.whole(seqs), trace_tools.decode_tail(seqs, tail=40))):
        got = trace_tools.run_inprocess(runner, tr, str(tmp_path / f"o{k}"))
        trace_tools.compare(tr, got, want, TOL[dtype])
    all_free(runner)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P", "Q"])
def test_portions_down_to_two_tokens(models, name, dtype, tmp_path):
    folder, cfg, w, seqs, want = models[name, dtype]
    runner = make_runner(folder, dtype, held(seqs))
    for k, sizes in enumerate(((7, 2, 24, 3, 2, 16, 5, 2, 31, 2), (2,), (64, 1, 3))):
        tr = trace_tools.portions(seqs, sizes=sizes)
        got = trace_tools.run_inprocess(runner, tr, str(tmp_path / f"o{k}"))
        trace_tools.compare(tr, got, want, TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P", "Q"])
def test_mixed_batches_with_pages_and_slots_used_again(models, name, dtype, tmp_path):
    """Unequal requests side by side, portions beside single tokens, in a pool of about two of the longest and
    with three state slots: every page and slot serves several requests in turn.  A state that is not zeroed
    at hand-out, or a row read from a page's former owner, shows against the plain statement."""
    folder, cfg, w, seqs, want = models[name, dtype]
    seqs2, want2 = seqs + seqs[::-1], want + want[::-1]
    max_tokens = 2 * held(seqs)
    runner = make_runner(folder, dtype, max_tokens, max_requests=3)
    tr = trace_tools.mixed(seqs2, max_tokens, seed=11, max_live=3)
    assert sum(len(s["entries"]) > 1 for s in tr.steps) > 5
    got = trace_tools.run_inprocess(runner, tr, str(tmp_path))
    trace_tools.compare(tr, got, want2, TOL[dtype])
    all_free(runner)


def test_a_request_alone_and_in_a_batch_agree(models, tmp_path):
    """float32: the same rows from a batch of unequal requests and from each request alone differ by rounding
    of sums at most (far less than from the plain statement)."""
    folder, cfg, w, seqs, want = models["P", "float32"]
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
    """Two tokens of prompt, then 300 tokens one by one across many pages: the recurrent state is carried 300 times,
    the attention's keys grow from 1; the first positions are compared one by one."""
    folder, cfg, w, _, _ = models["Q", dtype]
    rng = random.Random(77)
    seq = [rng.randrange(cfg["vocab"]) for _ in range(302)]
    want = expected(cfg, w, [seq])
    runner = make_runner(folder, dtype, 320)
    tr = trace_tools.decode_tail([seq], tail=300)
    got = trace_tools.run_inprocess(runner, tr, str(tmp_path))
    trace_tools.compare(tr, got, want, TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_one_far_key_stands_out(dtype, tmp_path):
    """Attention among hundreds of keys with one that matters: the queries are scaled up so that the softmax picks
    single keys (the plain statement confirms that most weight sits on one key, often far back).  A key that is
    lost, read from the wrong row of a page, or one position off changes the logits by far more than the tolerance.
    Prompts end just before, at and just after page borders; the tail is decoded token by token."""
    mix = zc.latent(4, 16, 8, 16, 32, 32, base=200.0, scale=1.0)
    cfg = zc.one_layer(mix, None, vocab=400, width=48)

    # bfloat16 rounds q and the cached rows to 8 bits: scores of this size then move by tenths, and so would the
    # weights of a softmax as sharp as the float32 run's; its run is a little less sharp
    factor, peak = (6.0, 0.5) if dtype == "float32" else (2.5, 0.2)

    def sharpen(t):
        t["l0.mix.uq"] = (t["l0.mix.uq"].float() * factor).to(torch.bfloat16)
    folder = zc.make_folder(cfg, str(tmp_path / "m"), seed=5, std=0.2, edit=sharpen)
    cfg, w = zc.read_folder(folder)
    rng = random.Random(8)
    seqs = [[rng.randrange(cfg["vocab"]) for _ in range(n)] for n in (255, 256, 257, 400)]
    # how peaked the plain statement's attention is, and how far back its strongest keys lie
    t64 = {k: v.to(torch.float64) for k, v in w.items()}
    x = pz.embed(t64["embed"], seqs[3], cfg["embedding"]["scale"])
    h = pz.offset_norm(x, t64["l0.norm1"], cfg["norm"]["eps"])
    m = cfg["layers"][0]["mixer"]
    short = {k[len("l0.mix."):]: v for k, v in t64.items() if k.startswith("l0.mix.")}
    T = len(seqs[3])
    cq = pz.plain_norm(h @ short["dq"].t(), short["dq.norm"], cfg["norm"]["eps"])
    q = (cq @ short["uq"].t()).view(T, m["heads"], -1)
    ckv = h @ short["dkv"].t()
    c = pz.plain_norm(ckv[:, :m["kv_rank"]], short["dkv.norm"], cfg["norm"]["eps"])
    kn = (c @ short["uk"].t()).view(T, m["heads"], m["dim"])
    pos = torch.arange(T)
    qr = pz.rotate_pairs(q[..., m["dim"]:], pos, m["rot"]["base"], m["rot"]["dims"])
    kr = pz.rotate_pairs(ckv[:, m["kv_rank"]:], pos, m["rot"]["base"], m["rot"]["dims"])
    s = (torch.einsum("ihd,jhd->hij", q[..., :m["dim"]], kn) + torch.einsum("ihd,jd->hij", qr, kr)) * m["scale"]
    s = s.masked_fill(pos[None, :] > pos[:, None], float("-inf"))
    p = torch.softmax(s, dim=-1)[:, 200:, :]
    top_p, top_j = p.max(dim=-1)
    assert float(top_p.median()) > peak                                   # one key carries most of the weight
    assert float(((pos[200:][None, :] - top_j) > 100).float().mean()) > 0.2    # and it is often far back
    want = expected(cfg, w, seqs)
    runner = make_runner(folder, dtype, 512)
    for k, tr in enumerate((trace_tools.whole(seqs), trace_tools.decode_tail(seqs, tail=24),
                            trace_tools.portions(seqs, sizes=(100, 2, 3, 64)))):
        got = trace_tools.run_inprocess(runner, tr, str(tmp_path / f"o{k}"))
        trace_tools.compare(tr, got, want, TOL[dtype])


def test_greedy_generation_through_the_engine(models):
    """``Engine.generate`` (scheduler, portions of prompts, batched decoding as replayed graphs, the sampler's
    argmax) against greedy decoding with the plain statement, for prompts of unequal length at once."""
    from qwen_decoder_b200.engine import Engine, SamplingParams
    folder, cfg, w, seqs, _ = models["P", "float32"]
    prompts = [seqs[2], seqs[5][:20], seqs[4], seqs[1], seqs[6][:50]]
    new = 12
    engine = Engine(folder, dtype="float32", max_batch=3, max_prefill_tokens_per_step=24, max_total_tokens=64,
                    num_pages=40, page_size=16, max_positions=256)
    outs = engine.generate(prompts, SamplingParams(max_new_tokens=new, ignore_eos=True))
    for prompt, out in zip(prompts, outs):
        seq = list(prompt)
        for _ in range(new):
            logits = pz.forward(cfg, w, seq)[-1]
            top2 = torch.topk(logits, 2).values
            assert float(top2[0] - top2[1]) > 1e-4, "a close call: choose another seed for this test"
            seq.append(int(torch.argmax(logits)))
        assert out == seq[len(prompt):]
    all_free(engine.runner)
    # bfloat16 with graphs: the same tokens whether a request runs alone or beside others
    folder = models["P", "bfloat16"][0]
    e16 = Engine(folder, dtype="bfloat16", max_batch=4, max_prefill_tokens_per_step=32, max_total_tokens=64,
                 num_pages=40, page_size=16, max_positions=256)
    together = e16.generate(prompts[:4], SamplingParams(max_new_tokens=new, ignore_eos=True))
    alone = [e16.generate([p], SamplingParams(max_new_tokens=new, ignore_eos=True))[0] for p in prompts[:4]]
    agree = sum(a == b for a, b in zip(together, alone))
    assert agree >= 3, (together, alone)       # a bfloat16 near-tie may flip one of them
