"""rutulix_oracle.py — plain, slow float64 statement of the Rutulix design (a layer-list model), for tests only.

One function per mechanism, written from the equations with numpy loops, token by token, and sharing no code with the CUDA
path.  `Sequence.feed` carries what a sequence carries: per layer run the list of all earlier (prepared key, value) pairs.

Notation: W x for a stored [out, in] matrix; ln(v) = (v - mean v) / sqrt(mean((v - mean v)^2) + eps) * w;
rms(v) = v / sqrt(mean(v^2) + eps) * w.

  model:      x = E[token];  layer runs in order;  logits = Hd ln_final(x)
  layer loop: layers start .. stop-1 run `times` times with the same weights; a layer run has its own keys and values;
              before pass t (also t = 0, also when times = 1) x <- x + step[t]
  layer:      x <- x + ln_1b(att(ln_1(x)));  x <- x + ln_2b(ff(ln_2(x)))   (no second line when the layer has no feed-forward)
  attention:  q = rms_q(W_q h) over all heads' rows at once, k = rms_k(W_k h) likewise; value of the position = W_k h itself;
              in every head the first `dims` entries are rotated pairwise (2i, 2i+1) by pos * f_i, scaled by the magnitude m;
              raw_g(j) = scale * q_g . k_j[g // (H/G)];  s_h(j) = sum_g talk[h, g] raw_g(j);
              p = softmax over the visible j (j <= pos and j // size == pos // size);  o_h = sum_j p_j v_j[h // (H/G)];  W_o concat(o)
  rotation:   f_i = base^(-2i/dims); with scaling {factor, original, fast, slow}:
              e(t) = dims * ln(original / (2 pi t)) / (2 ln base),  lo = max(floor e(fast), 0),  hi = min(ceil e(slow), dims - 1),
              r_i = clip((i - lo) / max(hi - lo, 0.001), 0, 1),  f_i <- r_i f_i / factor + (1 - r_i) f_i,  m = 0.1 ln(factor) + 1
  ff:         W_d a(W_u h + b_u) + b_d,  a(z) = sp(p) z^2 + z/2 for z > 0, (1/2 + sp(q)) (e^z - 1 - z) + z/2 otherwise, sp = log(1 + e^.)
"""
import math

import numpy as np

from hybrid_oracle import bf16_to_f64, to_bf16, write_checkpoint  # noqa: F401  (checkpoint minting helpers)


# ---- mechanisms -------------------------------------------------------------------------------------------------------
def layer_norm(v, w, eps):
    v = np.asarray(v, dtype=np.float64)
    d = v - v.mean()
    return d / math.sqrt(float(np.mean(d * d)) + eps) * w


def rms_norm(v, w, eps):
    v = np.asarray(v, dtype=np.float64)
    return v / math.sqrt(float(np.mean(v * v)) + eps) * w


def softplus(v):
    return np.logaddexp(0.0, v)


def rotation_table(rot):
    """Frequencies per pair and the magnitude factor of cos / sin."""
    dims, base = rot["dims"], rot["base"]
    f = np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)])
    mag = 1.0
    sc = rot.get("scaling")
    if sc:
        def e(t):
            return dims * math.log(sc["original"] / (2.0 * math.pi * t)) / (2.0 * math.log(base))
        lo, hi = max(math.floor(e(sc["fast"])), 0), min(math.ceil(e(sc["slow"])), dims - 1)
        for i in range(dims // 2):
            r = min(1.0, max(0.0, (i - lo) / max(hi - lo, 0.001)))
            f[i] = r * f[i] / sc["factor"] + (1.0 - r) * f[i]
        mag = 0.1 * math.log(sc["factor"]) + 1.0
    return f, mag


def rotate_heads(v, heads, dim, rot, pos):
    """v [heads * dim]: pairs (2i, 2i + 1) of the first rot["dims"] entries of every head turn by pos * f_i."""
    out = np.array(v, dtype=np.float64).reshape(heads, dim)
    if not rot or not rot.get("dims"):
        return out
    f, mag = rotation_table(rot)
    for h in range(heads):
        for i in range(rot["dims"] // 2):
            a = pos * f[i]
            c, s = math.cos(a) * mag, math.sin(a) * mag
            u, w = out[h, 2 * i], out[h, 2 * i + 1]
            out[h, 2 * i], out[h, 2 * i + 1] = u * c - w * s, w * c + u * s
    return out


def visible(mask, pos):
    """Positions j <= pos that position pos sees."""
    if not mask or "size" not in mask:
        return range(0, pos + 1)
    return range((pos // mask["size"]) * mask["size"], pos + 1)


def attention_step(W, p, mx, h, pos, keys, values, eps):
    """One token through the attention mixer; keys / values: lists over all earlier positions, appended here."""
    H, G, D = mx["heads"], mx["kv_heads"], mx["dim"]
    q = rms_norm(W[p + "q"] @ h, W[p + "q.norm"], eps)
    kraw = W[p + "k"] @ h
    k = rms_norm(kraw, W[p + "k.norm"], eps)
    keys.append(rotate_heads(k, G, D, mx.get("rot"), pos))
    values.append(kraw.reshape(G, D).copy())
    q = rotate_heads(q, H, D, mx.get("rot"), pos)
    js = list(visible(mx.get("mask"), pos))
    raw = np.zeros((H, len(js)))
    for g in range(H):
        for n, j in enumerate(js):
            raw[g, n] = mx["scale"] * float(q[g] @ keys[j][g // (H // G)])
    s = W[p + "talk"] @ raw
    out = np.zeros((H, D))
    for hh in range(H):
        e = np.exp(s[hh] - s[hh].max())
        pr = e / e.sum()
        for n, j in enumerate(js):
            out[hh] += pr[n] * values[j][hh // (H // G)]
    return W[p + "o"] @ out.reshape(-1), (js, s)


def xielu(z, p, q):
    z = np.asarray(z, dtype=np.float64)
    pos = softplus(p) * z * z + z / 2
    neg = (0.5 + softplus(q)) * (np.expm1(np.minimum(z, 0.0)) - z) + z / 2
    return np.where(z > 0, pos, neg)


def dense_ff(W, p, h):
    a = xielu(W[p + "up"] @ h + W[p + "up.b"], W[p + "act"][0], W[p + "act"][1])
    return W[p + "down"] @ a + W[p + "down.b"]


def layer_runs(cfg):
    """[(layer, pass or None)]: pass is set on the run that opens a pass of the loop."""
    n, lp = len(cfg["layers"]), cfg.get("loop")
    if not lp or lp["times"] < 1 or lp["stop"] <= lp["start"]:
        return [(i, None) for i in range(n)]
    runs = [(i, None) for i in range(lp["start"])]
    for t in range(lp["times"]):
        runs += [(i, t if i == lp["start"] else None) for i in range(lp["start"], lp["stop"])]
    return runs + [(i, None) for i in range(lp["stop"], n)]


# ---- a sequence -------------------------------------------------------------------------------------------------------
class Sequence:
    def __init__(self, cfg, W):
        self.cfg, self.W, self.eps = cfg, W, cfg["norm"]["eps"]
        self.runs = layer_runs(cfg)
        self.keys = [[] for _ in self.runs]
        self.values = [[] for _ in self.runs]
        self.pos = 0

    def feed(self, token, layers_out=None):
        cfg, W, eps = self.cfg, self.W, self.eps
        x = W["embed"][token].copy()
        for r, (i, t) in enumerate(self.runs):
            if t is not None:
                x = x + W["loop.step"][t]
            lc, p = cfg["layers"][i], f"l{i}."
            a, _ = attention_step(W, p + "mix.", lc["mixer"], layer_norm(x, W[p + "norm1"], eps), self.pos, self.keys[r], self.values[r], eps)
            x = x + layer_norm(a, W[p + "norm1b"], eps)
            if lc.get("mlp"):
                x = x + layer_norm(dense_ff(W, p + "mlp.", layer_norm(x, W[p + "norm2"], eps)), W[p + "norm2b"], eps)
            if layers_out is not None:
                layers_out.append(x.copy())
        self.pos += 1
        return W["head"] @ layer_norm(x, W["final.norm"], eps)


def run(cfg, W, tokens):
    """Logits [n, vocab] and residual traces [layer runs, n, width] of a whole sequence."""
    seq = Sequence(cfg, W)
    logits, traces = [], []
    for t in tokens:
        lo = []
        logits.append(seq.feed(int(t), lo))
        traces.append(lo)
    return np.array(logits), np.array(traces).transpose(1, 0, 2)


# ---- synthetic checkpoints ------------------------------------------------------------------------------------------------
def tensor_shapes(cfg):
    Wd, V = cfg["width"], cfg["vocab"]
    shapes = {"embed": (V, Wd), "final.norm": (Wd,), "head": (V, Wd)}
    lp = cfg.get("loop")
    if lp and lp["times"] >= 1:
        shapes["loop.step"] = (lp["times"], Wd)
    for i, lc in enumerate(cfg["layers"]):
        p, mx = f"l{i}.", lc["mixer"]
        H, G, D, Vd = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
        shapes.update({p + "norm1": (Wd,), p + "norm1b": (Wd,), p + "mix.q": (H * D, Wd), p + "mix.k": (G * D, Wd), p + "mix.q.norm": (H * D,),
                       p + "mix.k.norm": (G * D,), p + "mix.talk": (H, H), p + "mix.o": (Wd, H * Vd)})
        if lc.get("mlp"):
            ff = lc["mlp"]["ff"]
            shapes.update({p + "norm2": (Wd,), p + "norm2b": (Wd,), p + "mlp.up": (ff, Wd), p + "mlp.up.b": (ff,), p + "mlp.down": (Wd, ff),
                           p + "mlp.down.b": (Wd,), p + "mlp.act": (2,)})
    return shapes


def random_weights(cfg, seed=0):
    """bfloat16-representable random weights (as float64)."""
    rng = np.random.RandomState(seed)
    W = {}
    for name, shp in tensor_shapes(cfg).items():
        leaf = name.split(".")[-1]
        if leaf in ("norm1", "norm2", "norm") and not name.startswith("final"):
            a = 1.0 + 0.2 * rng.randn(*shp)
        elif leaf in ("norm1b", "norm2b"):
            a = 0.5 + 0.1 * rng.randn(*shp)
        elif name == "final.norm":
            a = 1.0 + 0.2 * rng.randn(*shp)
        elif leaf == "talk":
            a = np.eye(shp[0]) + 0.4 * rng.randn(*shp)
        elif leaf == "act":
            a = rng.uniform(-1.0, 1.0, shp)
        elif leaf == "b":
            a = 0.3 * rng.randn(*shp)
        elif name == "loop.step":
            a = 0.5 * rng.randn(*shp)
        elif name == "embed":
            a = rng.randn(*shp)
        else:
            a = 1.5 * rng.randn(*shp) / math.sqrt(shp[-1])
        W[name] = bf16_to_f64(to_bf16(a)).reshape(shp)
    return W


def att(heads=3, kv_heads=None, dim=8, size=6, scale=0.3, dims=4, base=100.0, scaling=None, ff=None):
    """One layer of a config."""
    rot = {"dims": dims, "base": base}
    if scaling:
        rot["scaling"] = scaling
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads or heads, "dim": dim, "vdim": dim, "scale": scale,
                                           "mask": {"size": size}, "rot": rot},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def model_config(layers, width=40, vocab=53, loop=None, eps=1e-5):
    cfg = {"architecture": "Rutulix", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": eps}}
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


def small_config():
    """A small model with every mechanism; sizes deliberately unequal from layer to layer and mostly not powers of two."""
    yarn = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}
    layers = [att(heads=6, kv_heads=2, dim=10, size=7, scale=0.3, dims=6, base=500.0, scaling=yarn, ff=28),
              att(heads=3, kv_heads=3, dim=12, size=19, scale=0.25, dims=12, base=1000.0, ff=None),
              att(heads=4, kv_heads=1, dim=6, size=5, scale=0.4, dims=2, base=50.0, scaling={"factor": 2.5, "original": 16, "fast": 4.0, "slow": 0.5}, ff=20),
              att(heads=2, kv_heads=2, dim=16, size=11, scale=0.2, dims=8, base=10000.0, ff=36)]
    return model_config(layers, width=44, vocab=61, loop=(1, 3, 3))
