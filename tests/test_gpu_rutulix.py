"""The Rutulix design in the layer-list family (sandwich blocks with layer norms, grouped-query attention whose values are the
key projection, whole-projection query / key norm, partial rotation with YaRN scaling, head mixing, chunk mask, dense xIELU
feed-forward, layer loop) against the plain float64 statement in oracle/rutulix_oracle.py.  Every test mints its own small
random checkpoint."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

F32_TOL = 2e-4


def rel(a, b):
    return float(np.abs(np.asarray(a, np.float64) - b).max() / max(np.abs(b).max(), 1e-30))


def close_bf16(a, b):
    """bfloat16 matrices against the float64 oracle, row by row (rounding is about 1e-3 of the scale for most rows)."""
    e = np.abs(np.asarray(a, np.float64) - b).max(-1) / max(np.abs(b).max(), 1e-30)
    return float(np.median(e)) < 1e-2 and float(np.quantile(e, 0.95)) < 3e-2 and float(e.max()) < 0.25


@pytest.fixture(scope="module")
def ro():
    import rutulix_oracle
    return rutulix_oracle


@pytest.fixture(scope="module")
def mk(tmp_path_factory, ro):
    """mk(cfg, seed, quant, chunk, context, edit) -> (dsk.Model, weights): mints the checkpoint, loads it through Model.from_dir."""
    import dsk
    root = tmp_path_factory.mktemp("rut")
    made, n = [], [0]

    def get(cfg, seed=0, quant="fp32", chunk=8, context=0, edit=None):
        W = ro.random_weights(cfg, seed)
        if edit:
            edit(W)
            W = {k: ro.bf16_to_f64(ro.to_bf16(v)).reshape(v.shape) for k, v in W.items()}
        n[0] += 1
        d = ro.write_checkpoint(str(root / f"m{n[0]}"), cfg, W)
        m = dsk.Model.from_dir(d, quant=quant, chunk=chunk, context=context)
        made.append(m)
        m.dir = d
        return m, W

    yield get
    for m in made:
        m.close()


def tokens_for(cfg, n, seed=0):
    return np.random.RandomState(seed).randint(0, cfg["vocab"], n).astype(np.int32)


def identity_talk(W):
    for k in W:
        if k.endswith("mix.talk"):
            W[k][:] = np.eye(W[k].shape[0])


def peaky(W):
    for k in W:
        if k.endswith("mix.q.norm"):
            W[k] *= 8.0          # scores x 8: a few keys take nearly all the weight, so a wrong edge or a lost key moves the output by O(1)


# ---- each mechanism alone -------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("kind", ["plain", "talk", "rotation", "rotation_full", "yarn", "yarn_step", "grouped", "chunks", "ff", "loop"])
def test_mechanism_alone(mk, ro, kind):
    """From one head group, no rotation, one chunk, identity head mixing, no feed-forward and no loop, one mechanism at a time."""
    a = dict(heads=3, kv_heads=3, dim=8, size=64, scale=0.3, dims=0, base=100.0)
    loop, edit = None, identity_talk
    if kind == "talk":
        edit = None
    elif kind == "rotation":
        a.update(dims=4)
    elif kind == "rotation_full":
        a.update(dims=8, base=7.0)
    elif kind == "yarn":
        a.update(dims=6, base=300.0, scaling={"factor": 6.0, "original": 32, "fast": 6.0, "slow": 0.75})
    elif kind == "yarn_step":      # both ends of the ramp fall on pair 0: the ramp is a step (the guard against a zero-length ramp)
        a.update(dims=8, base=1000.0, scaling={"factor": 16.0, "original": 8, "fast": 32.0, "slow": 2.0})
    elif kind == "grouped":
        a.update(heads=6, kv_heads=2)
    elif kind == "chunks":
        a.update(size=5)
    elif kind == "ff":
        a.update(ff=24)
    layers = [ro.att(**a)]
    if kind == "loop":
        layers, loop = [ro.att(**a), ro.att(**dict(a, heads=2, kv_heads=2))], (0, 1, 3)
    cfg = ro.model_config(layers, loop=loop)
    m, W = mk(cfg, seed=3, chunk=16, edit=edit)
    toks = tokens_for(cfg, 14, 1)
    exp, exp_layers = ro.run(cfg, W, toks)
    got, got_layers = m.forward_chunk(toks, 0, range(len(toks)), layers=True)
    assert got_layers.shape == exp_layers.shape
    assert rel(got_layers, exp_layers) < F32_TOL
    assert rel(got, exp) < F32_TOL


def test_yarn_table_changes_the_result(mk, ro):
    """The scaled frequencies and the magnitude factor are not a no-op: the same weights without scaling give other logits."""
    sc = {"factor": 6.0, "original": 32, "fast": 6.0, "slow": 0.75}
    f0, m0 = ro.rotation_table({"dims": 6, "base": 300.0})
    f1, m1 = ro.rotation_table({"dims": 6, "base": 300.0, "scaling": sc})
    assert m0 == 1.0 and m1 > 1.1 and f1[0] == f0[0] and f1[2] < f0[2] / 5.5 and f0[1] / 6 < f1[1] < f0[1]    # ramp 0, between, 1
    cfg_a = ro.model_config([ro.att(dims=6, base=300.0, scaling=sc, size=32)])
    cfg_b = ro.model_config([ro.att(dims=6, base=300.0, size=32)])
    toks = tokens_for(cfg_a, 20, 2)
    ma, W = mk(cfg_a, seed=4)
    mb, _ = mk(cfg_b, seed=4)
    ea, eb = ro.run(cfg_a, W, toks)[0], ro.run(cfg_b, W, toks)[0]
    assert rel(ma.forward_chunk(toks, 0, range(20)), ea) < F32_TOL and rel(mb.forward_chunk(toks, 0, range(20)), eb) < F32_TOL
    assert rel(ea, eb) > 1e-2


def test_activation_both_branches(ro):
    z = np.array([-3.0, -0.5, 0.0, 0.5, 3.0])
    out = ro.xielu(z, 0.3, -0.2)
    sp = lambda v: np.log1p(np.exp(v))
    assert np.allclose(out[3:], sp(0.3) * z[3:] ** 2 + z[3:] / 2)
    assert np.allclose(out[:3], (0.5 + sp(-0.2)) * (np.exp(z[:3]) - 1 - z[:3]) + z[:3] / 2)


# ---- schedules: whole prompt, token by token, portions ------------------------------------------------------------------------
@pytest.fixture(scope="module")
def full(mk, ro):
    cfg = ro.small_config()
    m, W = mk(cfg, seed=11, chunk=8)
    toks = tokens_for(cfg, 70, 4)
    exp, exp_layers = ro.run(cfg, W, toks)
    return cfg, m, W, toks, exp, exp_layers


def test_whole_prompt(full):
    cfg, m, W, toks, exp, exp_layers = full
    got, got_layers = m.forward_chunk(toks, 0, range(len(toks)), layers=True)   # 70 tokens = 9 internal steps of 8
    assert got_layers.shape[0] == 4 + 2 * 2                                       # two looped layers run three times
    assert rel(got_layers, exp_layers) < F32_TOL
    assert rel(got, exp) < F32_TOL


def test_token_by_token_equals_prefill(full):
    cfg, m, W, toks, exp, _ = full
    rows = [m.forward(int(t), i)[0].copy() for i, t in enumerate(toks)]
    assert rel(np.array(rows), exp) < F32_TOL


@pytest.mark.parametrize("chunk", [8, 64])      # steps below 32 tokens: the decode-sized kernel; 32 and more: the matrix-product path
@pytest.mark.parametrize("sizes", [[2] * 35, [3, 2, 5, 2, 7, 1, 8, 9, 2, 16, 2, 13], [33, 2, 35], [1, 69], [32, 38]])
def test_portions(mk, ro, full, chunk, sizes):
    cfg, _, W, toks, exp, _ = full
    m, _ = mk(cfg, seed=11, chunk=chunk)
    assert sum(sizes) == len(toks)
    p, rows = 0, []
    for c in sizes:
        rows.append(m.forward_chunk(toks[p:p + c], p, range(c)))
        p += c
    assert rel(np.concatenate(rows), exp) < F32_TOL


def test_decode_after_prompt(mk, full):
    cfg, _, W, toks, exp, _ = full
    m, _ = mk(cfg, seed=11, chunk=64)
    k = 37
    rows = [m.forward_chunk(toks[:k], 0, range(k))]
    rows += [m.forward_chunk(toks[i:i + 1], i, [0]) for i in range(k, len(toks))]
    assert rel(np.concatenate(rows), exp) < F32_TOL


def test_first_tokens_and_single_token_sequence(full, ro):
    cfg, m, W, toks, exp, _ = full
    for n in (1, 2, 3):
        assert rel(m.forward_chunk(toks[:n], 0, range(n)), exp[:n]) < F32_TOL
    one = ro.run(cfg, W, [7])[0]
    assert rel(m.forward_chunk([7], 0, [0]), one) < F32_TOL


# ---- states: interleaved sequences, states given back and used again ---------------------------------------------------
def test_interleaved_sequences_and_state_reuse(full, ro):
    cfg, m, W, toks, exp, _ = full
    other = tokens_for(cfg, 41, 9)
    exp_o = ro.run(cfg, W, other)[0]
    sa, sb = m.new_state(), m.new_state()
    ra, rb, pa, pb = [], [], 0, 0
    for ca, cb in [(5, 2), (1, 9), (17, 3), (2, 11), (45, 16)]:
        ra.append(m.forward_chunk(toks[pa:pa + ca], pa, range(ca), state=sa)); pa += ca
        rb.append(m.forward_chunk(other[pb:pb + cb], pb, range(cb), state=sb)); pb += cb
    assert rel(np.concatenate(ra), exp) < F32_TOL
    assert rel(np.concatenate(rb), exp_o) < F32_TOL
    # give both back and run each request in the other's state: nothing of the previous owner may show
    m.reset(state=sa); m.reset(state=sb)
    assert rel(m.forward_chunk(other, 0, range(len(other)), state=sa), exp_o) < F32_TOL
    assert rel(m.forward_chunk(toks, 0, range(len(toks)), state=sb), exp) < F32_TOL
    # position 0 starts a new sequence by itself; a shorter request after a longer one in the same state
    assert rel(m.forward_chunk(other[:9], 0, range(9), state=sb), exp_o[:9]) < F32_TOL


def test_loop_passes_keep_their_own_keys(mk, ro):
    """One looped layer: if the passes shared one cache, the keys of pass 0 would be overwritten by pass 1 before the next token
    reads them.  Also the pass vector: zeroing loop.step must change the result."""
    cfg = ro.model_config([ro.att(heads=2, dim=6, size=16, ff=12)], loop=(0, 1, 4), width=24)
    m, W = mk(cfg, seed=6, chunk=4)
    toks = tokens_for(cfg, 21, 3)
    exp, exp_layers = ro.run(cfg, W, toks)
    assert exp_layers.shape[0] == 4
    rows = [m.forward_chunk(toks[:5], 0, range(5))] + [m.forward_chunk(toks[i:i + 1], i, [0]) for i in range(5, 21)]
    assert rel(np.concatenate(rows), exp) < F32_TOL
    W0 = dict(W, **{"loop.step": np.zeros_like(W["loop.step"])})
    assert rel(ro.run(cfg, W0, toks)[0], exp) > 1e-2


# ---- chunk mask: edges, far keys, ring wrap ------------------------------------------------------------------------------------
@pytest.mark.parametrize("chunk", [8, 64])
@pytest.mark.parametrize("size", [1, 2, 5, 16])
def test_chunk_edge_sensitivity(mk, ro, size, chunk):
    """One attention layer: the logits at position i depend on exactly the tokens of its own chunk up to i.  Changing the last
    token of the chunk before must change nothing (bit for bit), changing the first token of the own chunk must; in prompts
    and in decoding; for a position at the start, in the middle and at the end of its chunk."""
    cfg = ro.model_config([ro.att(heads=4, kv_heads=2, size=size, ff=16)])
    m, W = mk(cfg, seed=21, chunk=chunk)
    n = 40

    def logits_at(toks, i, decode):
        if decode:
            m.forward_chunk(toks[:max(1, i - 6)], 0, [])
            for p in range(max(1, i - 6), i):
                m.forward_chunk(toks[p:p + 1], p, [])
            return m.forward_chunk(toks[i:i + 1], i, [0])[0]
        return m.forward_chunk(toks[:i + 1], 0, [i])[0]

    base = tokens_for(cfg, n, 5)
    for i in sorted({n - 1, (n // size) * size - 1, ((n - 1) // size) * size}):
        first = (i // size) * size
        for decode in (False, True):
            ref = logits_at(base, i, decode)
            outside = base.copy()
            outside[first - 1] = (outside[first - 1] + 1) % cfg["vocab"]
            assert np.array_equal(logits_at(outside, i, decode), ref)
            if first < i:
                inside = base.copy()
                inside[first] = (inside[first] + 1) % cfg["vocab"]
                assert np.abs(logits_at(inside, i, decode) - ref).max() > 1e-3


@pytest.mark.parametrize("chunk", [8, 64])
def test_chunk_edges_and_far_key_vs_oracle(mk, ro, chunk):
    """Peaky attention (scores x 8) over chunks of 23 and 150 positions with unequal layers, so what one layer hides another
    passes on: dominant keys fall on every offset to step, ring and chunk borders, far back and next to the edge.  Prompt in
    uneven portions, then decoding across two chunk borders of the larger mask."""
    cfg = ro.model_config([ro.att(heads=3, size=23, dims=4), ro.att(heads=4, kv_heads=2, dim=6, size=150, scale=0.4, dims=6, base=30.0, ff=20)])
    m, W = mk(cfg, seed=23, chunk=chunk, edit=peaky)
    n = 330
    toks = tokens_for(cfg, n, 6)
    exp = ro.run(cfg, W, toks)[0]
    p, rows = 0, []
    for c in [7, 16, 2, 31, 9, 64, 23, 40]:
        rows.append(m.forward_chunk(toks[p:p + c], p, range(c))); p += c
    while p < n:
        rows.append(m.forward_chunk(toks[p:p + 1], p, [0])); p += 1
    assert rel(np.concatenate(rows), exp) < F32_TOL
    assert rel(m.forward_chunk(toks, 0, range(n)), exp) < F32_TOL


def test_far_key_dominates(mk, ro):
    """A single key 288 positions back, among hundreds, takes half of the softmax: query and key projections are made equal, so
    a token's query matches its own key (32 per head) far better than any other token's (about 6 +- 6), and the token occurs
    once before it is asked for again.  Losing that key (a wrong first row of the mask, a ring row reused too early) moves the
    logits by O(1); the oracle says what they must be."""
    cfg = ro.model_config([ro.att(heads=2, dim=32, size=300, dims=0, scale=1.0)], vocab=40)

    def edit(W):
        identity_talk(W)
        W["l0.mix.q"][:] = W["l0.mix.k"]
        W["l0.mix.k.norm"][:] = 1.0
        W["l0.mix.q.norm"][:] = 1.0
    m, W = mk(cfg, seed=33, chunk=16, edit=edit)
    toks = np.random.RandomState(1).randint(0, 39, 299).astype(np.int32)
    toks[10] = toks[-1] = 39                                   # the only earlier occurrence of the last token
    seq = ro.Sequence(cfg, W)
    rows = np.array([seq.feed(int(t)) for t in toks])
    h = ro.layer_norm(W["embed"][39], W["l0.norm1"], 1e-5)
    _, (js, s) = ro.attention_step(W, "l0.mix.", cfg["layers"][0]["mixer"], h, 298, list(seq.keys[0][:298]), list(seq.values[0][:298]), 1e-5)
    pr = np.exp(s[0] - s[0].max())
    pr /= pr.sum()
    assert js[0] == 0 and pr[10] > 0.4                         # the far key and the token's own key share the weight
    got = [m.forward_chunk(toks[:250], 0, [249])] + [m.forward_chunk(toks[i:i + 1], i, [0]) for i in range(250, 299)]
    assert rel(np.concatenate(got), rows[249:]) < F32_TOL      # decoded, the step size far below the mask's size
    assert rel(m.forward_chunk(toks, 0, [298]), rows[298:]) < F32_TOL
    m2, _ = mk(cfg, seed=33, chunk=128, edit=edit)             # in a prompt, through the matrix-product path
    assert rel(m2.forward_chunk(toks, 0, [298]), rows[298:]) < F32_TOL


def test_long_decoding_wraps_the_ring(mk, ro):
    """Steps of 2 tokens and a chunk mask of 5: the key ring has 6 rows, so 160 decoded tokens go round it many times."""
    cfg = ro.model_config([ro.att(heads=2, size=5, ff=12), ro.att(heads=4, kv_heads=1, dim=6, size=3)], loop=(0, 2, 2))
    m, W = mk(cfg, seed=29, chunk=2)
    toks = tokens_for(cfg, 160, 8)
    exp = ro.run(cfg, W, toks)[0]
    rows = [m.forward_chunk(toks[:3], 0, range(3))] + [m.forward_chunk(toks[i:i + 1], i, [0]) for i in range(3, 160)]
    assert rel(np.concatenate(rows), exp) < F32_TOL
    assert rel(m.forward_chunk(toks, 0, range(160)), exp) < F32_TOL


def test_context_limit_is_enforced(mk, ro):
    import dsk
    cfg = ro.model_config([ro.att(size=64)])
    m, W = mk(cfg, seed=1, chunk=8, context=20)       # the mask's chunk does not fit: the cache holds 20 positions and no more
    m.forward_chunk(tokens_for(cfg, 20), 0, [19])
    with pytest.raises(dsk.DskError):
        m.forward_chunk([1], 20, [0])


def test_bad_configs_are_refused(ro):
    import dsk
    cfg = ro.model_config([ro.att(heads=4, kv_heads=3)])  # query heads must split evenly over the key heads
    hc, sp = dsk.rutulix_from_config(cfg, quant="fp32")
    with pytest.raises(dsk.DskError):
        dsk.Model(hc, layers=sp)
    cfg = ro.model_config([ro.att()])
    cfg["layers"][0]["mixer"]["vdim"] = 5                 # values come out of the key matrix: a different value size is contradictory
    hc, sp = dsk.rutulix_from_config(cfg, quant="fp32")
    with pytest.raises(dsk.DskError):
        dsk.Model(hc, layers=sp)
    cfg = ro.model_config([ro.att()], loop=(0, 3, 2))     # a loop beyond the last layer
    hc, sp = dsk.rutulix_from_config(cfg, quant="fp32")
    with pytest.raises(dsk.DskError):
        dsk.Model(hc, layers=sp)


# ---- other sizes --------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("case", ["ones", "odd", "wide", "one_pass", "loop_inside", "loop_all"])
def test_other_sizes(mk, ro, case):
    loop = None
    if case == "ones":      # every count that can be 1 is 1
        layers, width, vocab, loop = [ro.att(heads=1, kv_heads=1, dim=2, size=1, dims=2, ff=1)], 3, 3, (0, 1, 2)
    elif case == "odd":     # nothing is a multiple of 4; three query heads per key head; rotation of one pair only
        layers, width, vocab = [ro.att(heads=9, kv_heads=3, dim=7, size=11, dims=2, ff=5), ro.att(heads=5, kv_heads=5, dim=3, size=7, dims=2, ff=None)], 42, 97
    elif case == "wide":    # larger sizes: 16 heads of 64, 4 key heads, a mask wider than the prompt, full rotation
        layers, width, vocab = [ro.att(heads=16, kv_heads=4, dim=64, size=128, dims=64, base=10000.0, scale=0.125, ff=320),
                                ro.att(heads=8, kv_heads=8, dim=32, size=16, dims=16, scale=0.2, ff=96)], 192, 300
    else:
        layers, width, vocab = [ro.att(heads=2, size=4, ff=12), ro.att(heads=3, dim=6, size=9), ro.att(heads=2, kv_heads=1, dim=10, size=6, ff=8),
                                ro.att(heads=4, kv_heads=2, size=3, ff=10)], 36, 50
        loop = {"one_pass": (2, 3, 1), "loop_inside": (1, 3, 2), "loop_all": (0, 4, 2)}[case]   # one pass: no repeat, but its pass vector
    cfg = ro.model_config(layers, width=width, vocab=vocab, loop=loop)
    m, W = mk(cfg, seed=31, chunk=16)
    toks = tokens_for(cfg, 45, 3)
    exp, exp_layers = ro.run(cfg, W, toks)
    got, got_layers = m.forward_chunk(toks, 0, range(45), layers=True)
    assert rel(got_layers, exp_layers) < F32_TOL
    assert rel(got, exp) < F32_TOL
    rows = [m.forward_chunk(toks[:20], 0, range(20))] + [m.forward_chunk(toks[i:i + 1], i, [0]) for i in range(20, 45)]
    assert rel(np.concatenate(rows), exp) < F32_TOL
    if case == "ones":      # a layer norm over three values turns rounding into sign flips: no bfloat16 comparison here
        return
    mb, _ = mk(cfg, seed=31, chunk=64, quant="bf16")            # the bfloat16 kernels on the same sizes, matrix-product attention
    assert close_bf16(mb.forward_chunk(toks, 0, range(45)), exp)
    rows = [mb.forward_chunk(toks[:20], 0, range(20))] + [mb.forward_chunk(toks[i:i + 1], i, [0]) for i in range(20, 45)]
    assert close_bf16(np.concatenate(rows), exp)


def test_large_steps_and_many_wanted_rows(mk, ro):
    """A step above 256 tokens with every row wanted: two blocks of queries in the matrix-product attention, the second seeing
    keys of the first; the LM head runs over the wanted rows in several groups."""
    cfg = ro.model_config([ro.att(heads=4, kv_heads=2, size=200, ff=24), ro.att(size=50)], loop=(0, 1, 2))
    toks = tokens_for(cfg, 330, 7)
    for quant in ("fp32", "bf16"):
        m, W = mk(cfg, seed=41, chunk=512, quant=quant)
        exp = ro.run(cfg, W, toks)[0]
        ok = (lambda a, b: rel(a, b) < F32_TOL) if quant == "fp32" else close_bf16
        assert ok(m.forward_chunk(toks, 0, range(330)), exp)
        assert ok(m.forward_chunk(toks[:300], 0, [0, 150, 299]), exp[[0, 150, 299]])


def test_bf16_matrices(mk, ro):
    cfg = ro.small_config()
    m, W = mk(cfg, seed=11, quant="bf16", chunk=8)
    toks = tokens_for(cfg, 50, 4)
    exp = ro.run(cfg, W, toks)[0]
    assert close_bf16(m.forward_chunk(toks, 0, range(50)), exp)
    rows = [m.forward_chunk(toks[:30], 0, range(30))] + [m.forward_chunk(toks[i:i + 1], i, [0]) for i in range(30, 50)]
    assert close_bf16(np.concatenate(rows), exp)


# ---- generation through the framework's own entry points -------------------------------------------------------------------------
def oracle_greedy(ro, cfg, W, prompt, steps):
    seq = ro.Sequence(cfg, W)
    for t in prompt:
        lg = seq.feed(int(t))
    out, margins = [], []
    for _ in range(steps):
        top = np.sort(lg)[-2:]
        margins.append(top[1] - top[0])
        out.append(int(np.argmax(lg)))
        lg = seq.feed(out[-1])
    return out, min(margins)


def test_greedy_generation(full, ro):
    cfg, m, W, toks, exp, _ = full
    prompt, steps = toks[:12], 24
    want, margin = oracle_greedy(ro, cfg, W, prompt, steps)
    m.forward_chunk(prompt, 0, [len(prompt) - 1])
    dev, _ = m.decode_greedy(len(prompt), steps)                # device loop: a captured step, arg-max fed back without the host
    m.forward_chunk(prompt, 0, [len(prompt) - 1])
    host = []
    for i in range(steps):                                      # the samplers' loop: dsk_sample -> dsk_forward
        host.append(m.sample(temperature=0.0))
        m.forward(host[-1], len(prompt) + i)
    assert list(dev) == host
    if margin > 1e-3:                                           # no near-tie along the way: the oracle must agree token for token
        assert host == want


def test_cli_completion(full, repo):
    cfg, m, W, toks, exp, _ = full
    exe = os.path.join(repo, "deepseek.cpp_b200", "main")
    if not os.path.exists(exe):
        subprocess.check_call(["make", "-C", os.path.join(repo, "deepseek.cpp_b200"), "main"], stdout=subprocess.DEVNULL)
    prompt, steps = [int(t) for t in toks[:9]], 10
    r = subprocess.run([exe, m.dir, "-I", ",".join(map(str, prompt)), "-q", "fp32", "-n", str(steps), "-t", "0"], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    ids = [int(x) for x in r.stdout.split("generated ids:")[1].split()]
    m.forward_chunk(prompt, 0, [len(prompt) - 1])
    dev, _ = m.decode_greedy(len(prompt), steps)
    assert ids == prompt + list(dev)


def test_trace_runner(full, repo, tmp_path):
    """bin/trace_run end to end: two requests in turn, portions, decoded tokens, a state given back and used again."""
    cfg, m, W, toks, exp, _ = full
    out = tmp_path / "out"
    out.mkdir()
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": [int(t) for t in toks[:33]], "want": [0, 32]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [int(t) for t in toks[33:35]], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": [int(toks[35])], "want": [0]}], "end": ["a"]},
             {"step": 3, "entries": [{"id": "b", "tokens": [int(t) for t in toks[:8]], "want": [7, 3]}], "end": ["b"]}]
    r = subprocess.run([sys.executable, os.path.join(repo, "bin", "trace_run"), "--model", m.dir, "--dtype", "float32", "--out", str(out),
                        "--max-tokens", "64"], input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2", "done 3"]
    V = cfg["vocab"]
    g0 = np.fromfile(out / "0.f32", dtype="<f4").reshape(-1, V)
    g2 = np.fromfile(out / "2.f32", dtype="<f4").reshape(-1, V)
    g3 = np.fromfile(out / "3.f32", dtype="<f4").reshape(-1, V)
    assert not (out / "1.f32").exists()
    assert rel(g0, exp[[0, 32]]) < F32_TOL and rel(g2, exp[[35]]) < F32_TOL and rel(g3, exp[[7, 3]]) < F32_TOL


# ---- random designs -----------------------------------------------------------------------------------------------------------------
def random_design(seed):
    import rutulix_oracle as ro
    rng = np.random.RandomState(seed)
    n = int(rng.randint(1, 5))
    layers = []
    for _ in range(n):
        G = int(rng.choice([1, 2, 3]))
        rep = int(rng.choice([1, 2, 4]))
        D = int(rng.choice([2, 4, 6, 10, 16]))
        dims = int(rng.choice([d for d in (0, 2, 4, 6, 10, 16) if d <= D]))
        sc = None
        if dims and rng.rand() < 0.6:
            sc = {"factor": float(rng.choice([2.0, 4.0, 16.0])), "original": int(rng.choice([8, 32, 256])), "fast": float(rng.choice([4.0, 16.0, 32.0])),
                  "slow": float(rng.choice([0.5, 1.0, 2.0]))}
        layers.append(ro.att(heads=G * rep, kv_heads=G, dim=D, size=int(rng.choice([1, 3, 8, 20, 33, 70])), scale=float(rng.uniform(0.1, 0.6)),
                             dims=dims, base=float(rng.choice([10.0, 1000.0, 50000.0])), scaling=sc,
                             ff=int(rng.randint(1, 40)) if rng.rand() < 0.7 else None))
    loop = None
    if rng.rand() < 0.7:
        a = int(rng.randint(0, n))
        loop = (a, int(rng.randint(a + 1, n + 1)), int(rng.randint(1, 4)))
    return ro.model_config(layers, width=int(rng.choice([8, 20, 36, 50])), vocab=int(rng.randint(5, 90)), loop=loop,
                           eps=float(rng.choice([1e-6, 1e-5, 1e-3])))


@pytest.mark.parametrize("seed", range(8))
def test_random_designs(mk, ro, seed):
    """Layer count and order, every size, masks, rotation and loop drawn at random; whole prompt, prompt + decoded tail, uneven
    portions (steps on both attention paths)."""
    cfg = random_design(100 + seed)
    m, W = mk(cfg, seed=seed, chunk=40)
    n = 90
    toks = tokens_for(cfg, n, seed)
    exp = ro.run(cfg, W, toks)[0]
    assert rel(m.forward_chunk(toks, 0, range(n)), exp) < F32_TOL
    rows = [m.forward_chunk(toks[:60], 0, range(60))] + [m.forward_chunk(toks[i:i + 1], i, [0]) for i in range(60, n)]
    assert rel(np.concatenate(rows), exp) < F32_TOL
    p, rows = 0, []
    for c in [3, 34, 2, 2, 17, 5, 27]:
        rows.append(m.forward_chunk(toks[p:p + c], p, range(c))); p += c
    assert rel(np.concatenate(rows), exp) < F32_TOL
