"""Layer-list model family (state-space mixers, sliding-window latent attention, routed feed-forward, per-layer token input)
against the plain float64 statement in oracle/hybrid_oracle.py.  Every test mints its own small random checkpoint."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

F32_TOL, BF16_TOL = 2e-4, 5e-2


def rel(a, b):
    return float(np.abs(np.asarray(a, np.float64) - b).max() / max(np.abs(b).max(), 1e-30))


def close_bf16(a, b):
    """bfloat16 products against the float64 oracle, row by row: rounding errors are about 1e-3 of the scale for most rows and
    several times that where a small norm or a sharp softmax magnifies them; a wrong kernel is off by O(1) everywhere."""
    e = np.abs(np.asarray(a, np.float64) - b).max(-1) / max(np.abs(b).max(), 1e-30)
    return float(np.median(e)) < 1e-2 and float(np.quantile(e, 0.95)) < 3e-2 and float(e.max()) < 0.25


@pytest.fixture(scope="module")
def ho():
    import hybrid_oracle
    return hybrid_oracle


@pytest.fixture(scope="module")
def mk(tmp_path_factory, ho):
    """mk(cfg, seed, quant, chunk, edit=None) -> (dsk.Model, weights): mints the checkpoint, loads it through Model.from_dir."""
    import dsk
    root = tmp_path_factory.mktemp("hyb")
    made, n = [], [0]

    def get(cfg, seed=0, quant="fp32", chunk=8, context=0, edit=None):
        W = ho.random_weights(cfg, seed)
        if edit:
            edit(W)
            W = {k: ho.bf16_to_f64(ho.to_bf16(v)).reshape(v.shape) for k, v in W.items()}
        n[0] += 1
        d = ho.write_checkpoint(str(root / f"m{n[0]}"), cfg, W)
        m = dsk.Model.from_dir(d, quant=quant, chunk=chunk, context=context)
        made.append(m)
        m.dir = d
        return m, W

    yield get
    for m in made:
        m.close()


def ssd_layer(heads=3, vdim=10, state=12, groups=1, conv=3, ng=1, mlp=None, typ="mamba2"):
    return {"type": typ, "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": ng}, "mlp": mlp}


def att_layer(heads=3, dim=8, vdim=12, rank=20, win=6, scale=0.3, src=None, mlp=None):
    mx = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "mask": {"size": win}, "scale": scale}
    if src is not None:
        mx["kv_from"] = src
    return {"type": "latent_attention", "mixer": mx, "mlp": mlp}


def moe(E=6, top=2, ff=12, lim=1.5, sc=1.25):
    return {"kind": "moe", "router": {"experts": E, "top": top, "scale": sc}, "expert": {"ff": ff, "limit": lim}}


def model_cfg(layers, width=40, vocab=53, groups=2, side=0, m=0.7, ls=1.5):
    cfg = {"architecture": "Desarax", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": 1e-5, "groups": groups},
           "residual_mult": m, "logit_scale": ls}
    if side:
        cfg["token_side"] = {"dim": side}
    return cfg


def tokens_for(cfg, n, seed=0):
    return np.random.RandomState(seed).randint(0, cfg["vocab"], n).astype(np.int32)


# ---- each mechanism alone -------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("kind", ["ssd", "ssd_groups", "attention", "attention_shared", "moe", "side"])
def test_mechanism_alone(mk, ho, kind):
    layers = {"ssd": [ssd_layer()],
              "ssd_groups": [ssd_layer(heads=6, vdim=5, state=9, groups=3, conv=4, ng=2, typ="mamba2_2")],
              "attention": [att_layer()],
              "attention_shared": [att_layer(win=4), att_layer(heads=2, dim=6, vdim=5, win=9, scale=0.5, src=0)],
              "moe": [att_layer(win=1, mlp=moe())],
              "side": [ssd_layer()]}[kind]
    cfg = model_cfg(layers, side=5 if kind == "side" else 0)
    m, W = mk(cfg, seed=3, chunk=16)
    toks = tokens_for(cfg, 14, 1)
    exp, exp_layers = ho.run(cfg, W, toks)
    got, got_layers = m.forward_chunk(toks, 0, range(len(toks)), layers=True)
    assert rel(got_layers, exp_layers) < F32_TOL
    assert rel(got, exp) < F32_TOL


def test_router_choice_and_weights(mk, ho):
    """The selection uses score + correction, the weights the bare scores: a large correction must change who is chosen
    but not how the chosen are weighted."""
    cfg = model_cfg([att_layer(win=1, mlp=moe(E=8, top=3, sc=2.0))])

    def edit(W):
        W["l0.mlp.correction"][:] = 0.0
        W["l0.mlp.correction"][5] = 4.0          # expert 5 is always chosen, whatever its score
    m, W = mk(cfg, seed=5, edit=edit)
    toks = tokens_for(cfg, 9, 2)
    exp, _ = ho.run(cfg, W, toks)
    assert rel(m.forward_chunk(toks, 0, range(9)), exp) < F32_TOL
    h = ho.grouped_rms(W["embed"][toks[0]], W["l0.norm1"], 2, 1e-5)
    _, pick, wts = ho.routed_ff(W, "l0.mlp.", cfg["layers"][0]["mlp"], h)
    assert 5 in pick and abs(wts.sum() - 2.0) < 1e-9


# ---- schedules: whole prompt, token by token, portions ------------------------------------------------------------------------
@pytest.fixture(scope="module")
def full(mk, ho):
    cfg = ho.small_config()
    m, W = mk(cfg, seed=11, chunk=8)
    toks = tokens_for(cfg, 70, 4)
    exp, exp_layers = ho.run(cfg, W, toks)
    return cfg, m, W, toks, exp, exp_layers


def test_whole_prompt(full):
    cfg, m, W, toks, exp, exp_layers = full
    got, got_layers = m.forward_chunk(toks, 0, range(len(toks)), layers=True)   # 70 tokens = 9 internal steps of 8
    assert rel(got_layers, exp_layers) < F32_TOL
    assert rel(got, exp) < F32_TOL


def test_token_by_token_equals_prefill(full):
    cfg, m, W, toks, exp, _ = full
    rows = [m.forward(int(t), i)[0].copy() for i, t in enumerate(toks)]
    assert rel(np.array(rows), exp) < F32_TOL


@pytest.mark.parametrize("sizes", [[2] * 35, [3, 2, 5, 2, 7, 1, 8, 9, 2, 16, 2, 13], [33, 2, 35], [1, 69]])
def test_portions(full, sizes):
    cfg, m, W, toks, exp, _ = full
    assert sum(sizes) == len(toks)
    p, rows = 0, []
    for c in sizes:
        rows.append(m.forward_chunk(toks[p:p + c], p, range(c)))
        p += c
    assert rel(np.concatenate(rows), exp) < F32_TOL


def test_decode_after_prompt(full):
    cfg, m, W, toks, exp, _ = full
    k = 37
    rows = [m.forward_chunk(toks[:k], 0, range(k))]
    rows += [m.forward_chunk(toks[i:i + 1], i, [0]) for i in range(k, len(toks))]
    assert rel(np.concatenate(rows), exp) < F32_TOL


def test_first_tokens_and_single_token_sequence(full, ho):
    cfg, m, W, toks, exp, _ = full
    for n in (1, 2, 3):
        assert rel(m.forward_chunk(toks[:n], 0, range(n)), exp[:n]) < F32_TOL
    one = ho.run(cfg, W, [7])[0]
    assert rel(m.forward_chunk([7], 0, [0]), one) < F32_TOL


# ---- states: interleaved sequences, states given back and used again ---------------------------------------------------
def test_interleaved_sequences_and_state_reuse(full, ho):
    cfg, m, W, toks, exp, _ = full
    other = tokens_for(cfg, 41, 9)
    exp_o = ho.run(cfg, W, other)[0]
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
    # position 0 starts a new sequence by itself
    assert rel(m.forward_chunk(other[:9], 0, range(9), state=sb), exp_o[:9]) < F32_TOL


def test_positions_must_follow(full):
    import dsk
    cfg, m, W, toks, exp, _ = full
    m.forward_chunk(toks[:5], 0, [])
    with pytest.raises(dsk.DskError):
        m.forward_chunk(toks[5:8], 7, [])       # a gap: the recurrent state cannot skip positions
    with pytest.raises(dsk.DskError):
        m.forward_chunk([cfg["vocab"]], 5, [])  # token out of range


# ---- windows: edges, far keys, ring wrap ------------------------------------------------------------------------------------------
def peaky(W):
    for k in W:
        if k.endswith("mix.q") or k.endswith("mix.uk"):
            W[k] *= 3.0          # scores x 9: the softmax is dominated by a few keys, so a wrong edge moves the output by O(1)


@pytest.mark.parametrize("chunk", [8, 64])     # small steps: the absorbed-query kernel; steps of 32 tokens and more: the matrix-product path
@pytest.mark.parametrize("win", [1, 2, 5, 16])
def test_window_edge_sensitivity(mk, win, chunk):
    """One attention layer, no recurrence: the logits at position i depend on exactly the tokens i - win + 1 .. i.  Changing the
    token just outside the window must change nothing, the one just inside must change the result; in prompts and in decoding."""
    cfg = model_cfg([att_layer(heads=2, win=win, rank=12)], groups=1)
    m, W = mk(cfg, seed=21, chunk=chunk)     # plain random weights: every key of the window carries a visible share
    n = 40
    base = tokens_for(cfg, n, 5)
    i = n - 1

    def last_logits(toks, decode):
        if decode:
            m.forward_chunk(toks[:n - 6], 0, [])
            for p in range(n - 6, n - 1):
                m.forward_chunk(toks[p:p + 1], p, [])
            return m.forward_chunk(toks[n - 1:], n - 1, [0])[0]
        return m.forward_chunk(toks, 0, [n - 1])[0]

    for decode in (False, True):
        ref = last_logits(base, decode)
        outside, inside = base.copy(), base.copy()
        outside[i - win] = (outside[i - win] + 1) % cfg["vocab"]
        inside[i - win + 1] = (inside[i - win + 1] + 1) % cfg["vocab"]
        assert np.array_equal(last_logits(outside, decode), ref)
        assert np.abs(last_logits(inside, decode) - ref).max() > 1e-3


@pytest.mark.parametrize("chunk", [8, 64])
def test_window_edges_and_far_key_vs_oracle(mk, ho, chunk):
    """Peaky attention (scores x 9: one or two keys take nearly all the weight, wherever in the window they sit) over windows of
    23 and 150 tokens, the second reading the first one's latents, with a small step size: dominant keys fall on every offset to
    step, ring and window borders, far back and next to the edge.  Prompt in uneven portions, then decoding."""
    cfg = model_cfg([att_layer(heads=3, win=23, rank=16), ssd_layer(), att_layer(heads=2, dim=6, vdim=7, rank=16, win=150, scale=0.4, src=0)], groups=1)

    m, W = mk(cfg, seed=23, chunk=chunk, edit=peaky)
    n = 200
    toks = tokens_for(cfg, n, 6)
    exp = ho.run(cfg, W, toks)[0]
    p, rows = 0, []
    for c in [7, 16, 2, 31, 9, 64, 23]:
        rows.append(m.forward_chunk(toks[p:p + c], p, range(c))); p += c
    while p < n:
        rows.append(m.forward_chunk(toks[p:p + 1], p, [0])); p += 1
    assert rel(np.concatenate(rows), exp) < F32_TOL


def test_long_decoding_wraps_the_ring(mk, ho):
    """chunk 2 and window 5: the latent ring has 6 rows, so 160 decoded tokens go round it many times."""
    cfg = model_cfg([att_layer(heads=2, win=5, rank=12, mlp=moe(E=4, top=2)), ssd_layer(conv=2)], side=3)
    m, W = mk(cfg, seed=29, chunk=2)
    toks = tokens_for(cfg, 160, 8)
    exp = ho.run(cfg, W, toks)[0]
    rows = [m.forward_chunk(toks[:3], 0, range(3))] + [m.forward_chunk(toks[i:i + 1], i, [0]) for i in range(3, 160)]
    assert rel(np.concatenate(rows), exp) < F32_TOL
    assert rel(m.forward_chunk(toks, 0, range(160)), exp) < F32_TOL


def test_context_limit_is_enforced(mk):
    import dsk
    cfg = model_cfg([att_layer(win=64)])
    m, W = mk(cfg, seed=1, chunk=8, context=20)       # the window does not fit: the cache holds 20 positions and no more
    m.forward_chunk(tokens_for(cfg, 20), 0, [19])
    with pytest.raises(dsk.DskError):
        m.forward_chunk([1], 20, [0])


# ---- other sizes --------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("case", ["ones", "odd", "wide"])
def test_other_sizes(mk, ho, case):
    if case == "ones":      # every count that can be 1 is 1; no feed-forward in one layer, no token input, multipliers of 1
        cfg = model_cfg([ssd_layer(heads=1, vdim=1, state=1, groups=1, conv=1, ng=1), att_layer(heads=1, dim=1, vdim=1, rank=1, win=1, mlp=moe(E=1, top=1, ff=1)),
                         att_layer(heads=1, dim=2, vdim=1, rank=1, win=3, src=1)], width=4, vocab=3, groups=1, m=1.0, ls=1.0)
    elif case == "odd":     # nothing is a multiple of 4
        cfg = model_cfg([ssd_layer(heads=5, vdim=7, state=11, groups=5, conv=5, ng=5, mlp=moe(E=9, top=9, ff=7)),
                         att_layer(heads=7, dim=5, vdim=3, rank=33, win=11, mlp=moe(E=3, top=1, ff=5, lim=0.5))], width=42, vocab=97, groups=7, side=7)
    else:                   # larger powers of two: 512-thread scans, 8-register latent rows, 40 experts
        cfg = model_cfg([ssd_layer(heads=8, vdim=64, state=64, groups=2, conv=4, ng=4, mlp=moe(E=40, top=4, ff=64)),
                         att_layer(heads=9, dim=32, vdim=32, rank=160, win=40), ssd_layer(heads=2, vdim=80, state=136, groups=1),
                         att_layer(heads=4, dim=16, vdim=64, rank=160, win=64, src=1)], width=128, vocab=300, groups=4, side=16)
    m, W = mk(cfg, seed=31, chunk=16)
    toks = tokens_for(cfg, 45, 3)
    exp, exp_layers = ho.run(cfg, W, toks)
    got, got_layers = m.forward_chunk(toks, 0, range(45), layers=True)
    assert rel(got_layers, exp_layers) < F32_TOL
    assert rel(got, exp) < F32_TOL
    rows = [m.forward_chunk(toks[:20], 0, range(20))] + [m.forward_chunk(toks[i:i + 1], i, [0]) for i in range(20, 45)]
    assert rel(np.concatenate(rows), exp) < F32_TOL
    if case != "wide":      # the bfloat16 kernels on the same sizes: unaligned rows and K tails take their scalar paths
        mb, _ = mk(cfg, seed=31, chunk=64, quant="bf16")
        assert close_bf16(mb.forward_chunk(toks, 0, range(45)), exp)
        rows = [mb.forward_chunk(toks[:20], 0, range(20))] + [mb.forward_chunk(toks[i:i + 1], i, [0]) for i in range(20, 45)]
        assert close_bf16(np.concatenate(rows), exp)


def test_large_steps_and_many_wanted_rows(mk, ho):
    """A step size above 256 with every row wanted: the LM head runs over the wanted rows in several groups, the routed
    feed-forward sees full row tiles, the scan stages 64 tokens per round."""
    cfg = model_cfg([ssd_layer(mlp=moe(E=3, top=2)), att_layer(win=50)], side=4)
    toks = tokens_for(cfg, 330, 7)
    for quant in ("fp32", "bf16"):
        m, W = mk(cfg, seed=41, chunk=512, quant=quant)
        exp = ho.run(cfg, W, toks)[0]
        ok = (lambda a, b: rel(a, b) < F32_TOL) if quant == "fp32" else close_bf16
        assert ok(m.forward_chunk(toks, 0, range(330)), exp)
        assert ok(m.forward_chunk(toks[:300], 0, [0, 150, 299]), exp[[0, 150, 299]])


def test_bf16_matrices(mk, ho):
    cfg = ho.small_config()
    m, W = mk(cfg, seed=11, quant="bf16", chunk=8)
    toks = tokens_for(cfg, 50, 4)
    exp = ho.run(cfg, W, toks)[0]
    assert close_bf16(m.forward_chunk(toks, 0, range(50)), exp)
    rows = [m.forward_chunk(toks[:30], 0, range(30))] + [m.forward_chunk(toks[i:i + 1], i, [0]) for i in range(30, 50)]
    assert close_bf16(np.concatenate(rows), exp)


# ---- generation through the framework's own entry points -------------------------------------------------------------------------
def test_greedy_generation(full, ho):
    cfg, m, W, toks, exp, _ = full
    prompt, steps = toks[:12], 24
    m.forward_chunk(prompt, 0, [len(prompt) - 1])
    dev, _ = m.decode_greedy(len(prompt), steps)                # device loop: arg-max fed back without the host
    m.forward_chunk(prompt, 0, [len(prompt) - 1])
    host, t = [], m.sample(0.0)
    for i in range(steps):                                      # the CLI's loop: dsk_sample -> dsk_forward
        host.append(t)
        m.forward(t, len(prompt) + i)
        t = m.sample(0.0)
    assert dev.tolist() == host
    seq = ho.Sequence(cfg, W)
    for t in prompt:
        lg = seq.feed(int(t))
    for t in dev:                                               # each generated token is the oracle's arg-max (up to a near tie)
        assert lg[t] >= lg.max() - 1e-3 * np.abs(lg).max()
        lg = seq.feed(int(t))
    p = m.sample_prob(int(dev[-1]))
    assert 0.0 <= p <= 1.0


def test_trace_runner(full, ho, repo, tmp_path):
    cfg, m, W, toks, exp, _ = full
    other = tokens_for(cfg, 30, 12)
    exp_o = ho.run(cfg, W, other)[0]
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks[:33].tolist(), "want": [0, 32, 5]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": toks[33:35].tolist(), "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": toks[35:36].tolist(), "want": [0]}], "end": ["a"]},
             {"step": 3, "entries": [{"id": "b", "tokens": other.tolist(), "want": [29]}], "end": ["b"]},
             {"step": 4, "entries": [{"id": "c", "tokens": toks[:2].tolist(), "want": [1]}], "end": ["c"]}]
    for dtype, tol in (("float32", F32_TOL), ("bfloat16", BF16_TOL)):
        out = tmp_path / dtype
        out.mkdir()
        r = subprocess.run([os.path.join(repo, "bin", "trace_run"), "--model", m.dir, "--dtype", dtype, "--out", str(out), "--max-tokens", "64"],
                           input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        assert [l for l in r.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(5)]
        rd = lambda i: np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, cfg["vocab"])
        assert rel(rd(0), exp[[0, 32, 5]]) < tol
        assert not (out / "1.f32").exists()
        assert rel(rd(2), exp[[35]]) < tol
        assert rel(rd(3), exp_o[[29]]) < tol
        assert rel(rd(4), exp[[1]]) < tol


def test_cli_completion(full, repo):
    """The C++ host on a config.json checkpoint: prompt ids in (prefilled in portions), greedy ids out, equal to the device loop."""
    import re
    cfg, m, W, toks, exp, _ = full
    exe = os.path.join(repo, "deepseek.cpp_b200", "main")
    if not os.path.exists(exe):
        subprocess.check_call(["make", "-C", os.path.dirname(exe), "main"])
    prompt, steps = toks[:21].tolist(), 12
    out = subprocess.run([exe, m.dir, "-I", ",".join(map(str, prompt)), "-n", str(steps), "-t", "0", "-q", "fp32", "-T", "40"],
                         capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    ids = [int(v) for v in re.search(r"generated ids:([ 0-9]+)", out.stdout).group(1).split()]
    assert ids[:len(prompt)] == prompt and len(ids) == len(prompt) + steps
    m.forward_chunk(prompt, 0, [len(prompt) - 1])
    dev, _ = m.decode_greedy(len(prompt), steps)
    assert ids[len(prompt):] == dev.tolist()


def test_forward_chunk_on_deepseek_models(ckpt):
    """dsk_forward_chunk is the framework's portion call for every family: a DeepSeek model runs its hydrate loop inside it."""
    import dsk
    m = dsk.Model.from_dir(ckpt("tiny_v2lite", "fp32"))
    toks = [0, 17, 300, 5, 9]
    rows = [m.forward(t, i)[0].copy() for i, t in enumerate(toks)]
    got = m.forward_chunk(toks, 0, [1, 4])
    assert np.array_equal(got[0], rows[1]) and np.array_equal(got[1], rows[4])
    m.reset()
    assert np.array_equal(m.forward_chunk(toks[:2], 0, [1])[0], rows[1])
    m.close()


def random_design(seed):
    """A random model of the family: layer order, every size, windows, sharing of latent caches and constants drawn at random."""
    r = np.random.RandomState(seed)
    div = lambda n: int(r.choice([d for d in range(1, n + 1) if n % d == 0]))
    parts = lambda n: int(r.choice([d for d in range(1, n + 1) if n % d == 0 and (n // d >= 4 or d == 1)]))   # norm groups of 4 values and more:
    # a norm over one or two values is a sign function, which turns rounding noise into O(1) differences
    width = int(r.choice([24, 36, 40, 56, 72, 96, 130]))
    layers, owners = [], []
    for i in range(int(r.randint(2, 8))):
        ff = None
        if r.rand() < 0.7:
            E = int(r.randint(2, 21))
            ff = moe(E=E, top=int(r.randint(1, min(E, 4) + 1)), ff=int(r.randint(4, 50)), lim=float(r.uniform(0.5, 4.0)), sc=float(r.uniform(0.5, 2.5)))
        if r.rand() < 0.5:
            heads = int(r.randint(1, 9))
            vdim = int(r.randint(3, 41))
            layers.append(ssd_layer(heads=heads, vdim=vdim, state=int(r.randint(4, 71)), groups=div(heads), conv=int(r.randint(1, 6)),
                                    ng=parts(heads * vdim) if r.rand() < 0.5 else 1, mlp=ff, typ=str(r.choice(["mamba2", "mamba2_2"]))))
        else:
            src = None
            rank = int(r.randint(8, 101))
            if owners and r.rand() < 0.4:
                src = int(r.choice(owners))
                rank = layers[src]["mixer"]["kv_rank"]
            else:
                owners.append(i)
            layers.append(att_layer(heads=int(r.randint(1, 8)), dim=int(r.randint(4, 41)), vdim=int(r.randint(4, 41)), rank=rank,
                                    win=int(r.choice([1, 2, 3, 7, 16, 31, 32, 33, 50, 80])), scale=float(r.uniform(0.1, 0.6)), src=src, mlp=ff))
    return model_cfg(layers, width=width, vocab=int(r.randint(5, 200)), groups=parts(width) if r.rand() < 0.7 else 1,
                     side=int(r.randint(2, 13)) if r.rand() < 0.6 else 0, m=float(r.uniform(0.3, 1.0)), ls=float(r.uniform(0.5, 2.0)))


@pytest.mark.parametrize("seed", range(8))
def test_random_designs(mk, ho, seed):
    """Whole prompt, prompt + decoded tail, and uneven portions (both attention paths, the internal step boundary at 64) of a random
    design against the oracle, in fp32; then the bfloat16 kernels on the same model."""
    cfg = random_design(100 + seed)
    m, W = mk(cfg, seed=seed, chunk=64)
    n = 150
    toks = tokens_for(cfg, n, seed)
    exp = ho.run(cfg, W, toks)[0]
    assert rel(m.forward_chunk(toks, 0, range(n)), exp) < F32_TOL
    rows = [m.forward_chunk(toks[:110], 0, range(110))] + [m.forward_chunk(toks[i:i + 1], i, [0]) for i in range(110, n)]
    assert rel(np.concatenate(rows), exp) < F32_TOL
    r, p, rows = np.random.RandomState(seed), 0, []
    while p < n:
        c = min(int(r.choice([2, 3, 5, 17, 33, 40, 64, 70])), n - p)
        rows.append(m.forward_chunk(toks[p:p + c], p, range(c)))
        p += c
    assert rel(np.concatenate(rows), exp) < F32_TOL
    # bfloat16 matrices.  Steps of up to 4 tokens multiply them with the fp32 activations: the weights are exact in bfloat16, so
    # this path must agree as tightly as the fp32 one.  Larger steps round the activations to bfloat16 on the way into the tensor
    # cores: small random models magnify that (and a routed layer may flip a near-tied expert), so only the bulk is bounded —
    # a wrong kernel is off by O(1) in every row.
    mb, _ = mk(cfg, seed=seed, chunk=64, quant="bf16")
    rows, p = [], 0
    while p < 60:
        c = min(int(r.choice([1, 2, 3, 4])), 60 - p)
        rows.append(mb.forward_chunk(toks[p:p + c], p, range(c)))
        p += c
    assert rel(np.concatenate(rows), exp[:60]) < F32_TOL
    e = np.abs(mb.forward_chunk(toks, 0, range(n)) - exp).max(-1) / np.abs(exp).max()
    assert np.median(e) < 6e-2
