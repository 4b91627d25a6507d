"""hybrid_oracle.py — plain, slow float64 statement of the layer-list ("hybrid") model family, for tests only.

One function per mechanism, written from the equations (numpy loops, no batching tricks) and sharing no code with the CUDA
path.  A sequence is processed token by token through `Sequence.feed`, which carries exactly what the design says a sequence
carries: per state-space layer the matrix S and the last (taps - 1) convolution inputs, per latent-attention layer the
latents of all earlier positions.

Notation: W x for a stored [out, in] matrix W; rms(v) = v / sqrt(mean(v^2) + eps).

  layer:      h = grouped_rms(x) * w_norm1;  x <- x + m * (mixer(h) + ff(h))
              then (if the model has a per-layer token table of width sd):
              g = gelu_tanh(G x) * table[token, i*sd:(i+1)*sd];  y = P g;  x <- x + m * rms(y) * w_side
  ssd mixer:  [z | xBC | dt] = W_in h;  xBC <- silu(causal depthwise conv(xBC) + b);  dt <- log(1 + exp(dt + dt_bias))
              per head k (group k // (heads/groups)):  S <- exp(-exp(A_log_k) dt_k) S + dt_k B x_k^T;  y_k = S^T C + D_k x_k
              out = W_o (grouped_rms(y * silu(z)) * w_norm)
  latent att: c = rms(W_dkv h) * w_dkv (or another layer's cached c);  per head: k_j = W_uk c_j, v_j = W_uv c_j,
              p = softmax_j(scale * q . k_j) over 0 <= i - j < window;  out = W_o concat_heads(sum_j p_j v_j)
  routed ff:  s = sigmoid(W_r h); pick the `top` largest s + correction; w = s_picked / (sum s_picked + 1e-20) * scale;
              expert(h) = W_down (g * sigmoid(1.702 g) * (u + 1)),  g = min(W_gate h, limit),  u = clip(W_up h, -limit, limit)
  head:       logits = E (grouped_rms(x) * w_final) * logit_scale,  E the embedding table
"""
import json
import math
import os

import numpy as np


# ---- mechanisms -------------------------------------------------------------------------------------------------------
def grouped_rms(v, w, groups, eps):
    v = np.asarray(v, dtype=np.float64)
    out = np.empty_like(v)
    n = v.shape[0] // groups
    for g in range(groups):
        part = v[g * n:(g + 1) * n]
        out[g * n:(g + 1) * n] = part / math.sqrt(float(np.mean(part * part)) + eps)
    return out * w


def silu(v):
    return v / (1.0 + np.exp(-v))


def gelu_tanh(v):
    return 0.5 * v * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (v + 0.044715 * v ** 3)))


def softplus(v):
    return np.logaddexp(0.0, v)


def ssd_step(W, p, mx, h, carry, eps):
    """One token through a state-space mixer.  carry = {"S": [heads, state, vdim], "hist": [taps - 1, channels]}."""
    H, P, N, G, K = mx["heads"], mx["vdim"], mx["state"], mx.get("groups", 1), mx["conv"]
    inner, gn = H * P, G * N
    u = W[p + "in"] @ h
    z, xbc, dt = u[:inner], u[inner:2 * inner + 2 * gn], u[2 * inner + 2 * gn:]
    window = np.vstack([carry["hist"], xbc[None, :]])              # taps rows, oldest first; the last row is this token
    carry["hist"] = window[1:].copy()
    conv = silu((window * W[p + "conv"].T).sum(0) + W[p + "conv.b"])
    xs, B, C = conv[:inner].reshape(H, P), conv[inner:inner + gn].reshape(G, N), conv[inner + gn:].reshape(G, N)
    dt = softplus(dt + W[p + "dt_bias"])
    y = np.zeros((H, P))
    for k in range(H):
        g = k // (H // G)
        decay = math.exp(-math.exp(W[p + "A_log"][k]) * dt[k])
        carry["S"][k] = decay * carry["S"][k] + dt[k] * np.outer(B[g], xs[k])
        y[k] = carry["S"][k].T @ C[g] + W[p + "D"][k] * xs[k]
    gated = y.reshape(-1) * silu(z)
    return W[p + "o"] @ grouped_rms(gated, W[p + "norm"], mx.get("norm_groups", 1), eps)


def latent_of(W, p, h, eps):
    return grouped_rms(W[p + "dkv"] @ h, W[p + "dkv.norm"], 1, eps)


def latent_attention_step(W, p, mx, h, latents):
    """One token (the newest; its latent is latents[-1]) attending over the cached latents of its window."""
    H, D, V = mx["heads"], mx["dim"], mx["vdim"]
    win = (mx.get("mask") or {}).get("size")
    i = len(latents) - 1
    first = 0 if win is None else max(0, i - win + 1)
    q = (W[p + "q"] @ h).reshape(H, D)
    out = np.zeros((H, V))
    for k in range(H):
        Wk, Wv = W[p + "uk"][k * D:(k + 1) * D], W[p + "uv"][k * V:(k + 1) * V]
        scores = np.array([mx["scale"] * float(q[k] @ (Wk @ latents[j])) for j in range(first, i + 1)])
        e = np.exp(scores - scores.max())
        pr = e / e.sum()
        for n, j in enumerate(range(first, i + 1)):
            out[k] += pr[n] * (Wv @ latents[j])
    return W[p + "o"] @ out.reshape(-1)


def routed_ff(W, p, fc, h):
    top, scale, lim = fc["router"]["top"], fc["router"].get("scale", 1.0), fc["expert"]["limit"]
    s = 1.0 / (1.0 + np.exp(-(W[p + "router"] @ h)))
    pick = np.argsort(-(s + W[p + "correction"]), kind="stable")[:top]
    wts = s[pick] / (s[pick].sum() + 1e-20) * scale
    out = np.zeros_like(h)
    for e, wt in zip(pick, wts):
        g = np.minimum(W[f"{p}e{e}.gate"] @ h, lim)
        u = np.clip(W[f"{p}e{e}.up"] @ h, -lim, lim)
        out += wt * (W[f"{p}e{e}.down"] @ (g / (1.0 + np.exp(-1.702 * g)) * (u + 1.0)))
    return out, pick, wts


def token_side(W, p, x, row, eps):
    y = W[p + "proj"] @ (gelu_tanh(W[p + "gate"] @ x) * row)
    return y / math.sqrt(float(np.mean(y * y)) + eps) * W[p + "norm"]


# ---- a sequence -------------------------------------------------------------------------------------------------------
class Sequence:
    def __init__(self, cfg, W):
        self.cfg, self.W = cfg, W
        self.eps = (cfg.get("norm") or {}).get("eps", 1e-5)
        self.groups = (cfg.get("norm") or {}).get("groups", 1)
        self.m = cfg.get("residual_mult", 1.0)
        self.carry = []
        for lc in cfg["layers"]:
            mx = lc["mixer"]
            if "state" in mx:
                ch = mx["heads"] * mx["vdim"] + 2 * mx.get("groups", 1) * mx["state"]
                self.carry.append({"S": np.zeros((mx["heads"], mx["state"], mx["vdim"])), "hist": np.zeros((mx["conv"] - 1, ch))})
            else:
                self.carry.append({"latents": []})

    def feed(self, token, layers_out=None):
        """One more token: returns its logits; layers_out (a list) receives the residual stream after every layer."""
        cfg, W = self.cfg, self.W
        x = W["embed"][token].copy()
        for i, lc in enumerate(cfg["layers"]):
            p, mx = f"l{i}.", lc["mixer"]
            h = grouped_rms(x, W[p + "norm1"], self.groups, self.eps)
            if "state" in mx:
                a = ssd_step(W, p + "mix.", mx, h, self.carry[i], self.eps)
            else:
                src = mx.get("kv_from")
                if src is None:
                    self.carry[i]["latents"].append(latent_of(W, p + "mix.", h, self.eps))
                    src = i
                a = latent_attention_step(W, p + "mix.", mx, h, self.carry[src]["latents"])
            f = routed_ff(W, p + "mlp.", lc["mlp"], h)[0] if lc.get("mlp") else 0.0
            x = x + self.m * (a + f)
            if cfg.get("token_side"):
                sd = cfg["token_side"]["dim"]
                x = x + self.m * token_side(W, p + "side.", x, W["side.embed"][token, i * sd:(i + 1) * sd], self.eps)
            if layers_out is not None:
                layers_out.append(x.copy())
        return (W["embed"] @ grouped_rms(x, W["final.norm"], self.groups, self.eps)) * cfg.get("logit_scale", 1.0)


def run(cfg, W, tokens):
    """Logits [n, vocab] and residual traces [layers, n, width] of a whole sequence."""
    seq = Sequence(cfg, W)
    logits, traces = [], []
    for t in tokens:
        lo = []
        logits.append(seq.feed(int(t), lo))
        traces.append(lo)
    return np.array(logits), np.array(traces).transpose(1, 0, 2)


# ---- synthetic checkpoints ------------------------------------------------------------------------------------------------
def to_bf16(a):
    """Round-to-nearest-even bfloat16 as uint16."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def bf16_to_f64(u):
    return (u.astype(np.uint32) << 16).view(np.float32).astype(np.float64)


def tensor_shapes(cfg):
    Wd, V = cfg["width"], cfg["vocab"]
    shapes = {"embed": (V, Wd), "final.norm": (Wd,)}
    sd = (cfg.get("token_side") or {}).get("dim", 0)
    if sd:
        shapes["side.embed"] = (V, sd * len(cfg["layers"]))
    for i, lc in enumerate(cfg["layers"]):
        p, mx = f"l{i}.", lc["mixer"]
        shapes[p + "norm1"] = (Wd,)
        if "state" in mx:
            H, P, N, G, K = mx["heads"], mx["vdim"], mx["state"], mx.get("groups", 1), mx["conv"]
            inner, ch = H * P, H * P + 2 * G * N
            shapes.update({p + "mix.in": (inner + ch + H, Wd), p + "mix.conv": (ch, K), p + "mix.conv.b": (ch,), p + "mix.dt_bias": (H,),
                           p + "mix.A_log": (H,), p + "mix.D": (H,), p + "mix.norm": (inner,), p + "mix.o": (Wd, inner)})
        else:
            H, D, Vd, R = mx["heads"], mx["dim"], mx["vdim"], mx["kv_rank"]
            shapes.update({p + "mix.q": (H * D, Wd), p + "mix.uk": (H * D, R), p + "mix.uv": (H * Vd, R), p + "mix.o": (Wd, H * Vd)})
            if mx.get("kv_from") is None:
                shapes.update({p + "mix.dkv": (R, Wd), p + "mix.dkv.norm": (R,)})
        if lc.get("mlp"):
            E, ff = lc["mlp"]["router"]["experts"], lc["mlp"]["expert"]["ff"]
            shapes.update({p + "mlp.router": (E, Wd), p + "mlp.correction": (E,)})
            for e in range(E):
                shapes.update({f"{p}mlp.e{e}.gate": (ff, Wd), f"{p}mlp.e{e}.up": (ff, Wd), f"{p}mlp.e{e}.down": (Wd, ff)})
        if sd:
            shapes.update({p + "side.gate": (sd, Wd), p + "side.proj": (Wd, sd), p + "side.norm": (Wd,)})
    return shapes


def random_weights(cfg, seed=0):
    """bfloat16-representable random weights (as float64) of a size that keeps activations O(1)."""
    rng = np.random.RandomState(seed)
    W = {}
    for name, shp in tensor_shapes(cfg).items():
        leaf = name.split(".")[-1]
        if leaf in ("norm1", "norm") or name.endswith("dkv.norm"):
            a = 1.0 + 0.2 * rng.randn(*shp)
        elif leaf == "A_log":
            a = np.log(rng.uniform(0.3, 3.0, shp))
        elif leaf == "dt_bias":
            a = rng.uniform(-2.5, 0.5, shp)
        elif leaf == "D":
            a = rng.uniform(0.5, 1.5, shp)
        elif leaf == "b":
            a = 0.2 * rng.randn(*shp)
        elif leaf == "conv":
            a = 0.5 * rng.randn(*shp)
        elif leaf == "correction":
            a = 0.3 * rng.randn(*shp)
        elif name in ("embed", "side.embed"):
            a = rng.randn(*shp)
        elif leaf == "router":
            a = 2.0 * rng.randn(*shp) / math.sqrt(shp[1])
        else:
            a = 1.5 * rng.randn(*shp) / math.sqrt(shp[-1])
        W[name] = bf16_to_f64(to_bf16(a)).reshape(shp)
    return W


def write_checkpoint(dirname, cfg, W):
    """config.json + model.safetensors (bfloat16) in `dirname`."""
    import dseek
    os.makedirs(dirname, exist_ok=True)
    with open(os.path.join(dirname, "config.json"), "w") as f:
        json.dump(cfg, f, indent=1)
    dseek.write_shard(os.path.join(dirname, "model.safetensors"), {k: ("BF16", to_bf16(v).reshape(v.shape)) for k, v in W.items()})
    return dirname


def small_config(**kw):
    """A small model with every mechanism; sizes deliberately unequal and mostly not powers of two."""
    ssd = lambda heads, vdim, state, groups, conv, ng: {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups,
                                                                                    "conv": conv, "norm_groups": ng}}
    att = lambda heads, dim, vdim, rank, win, scale, src=None: {"type": "latent_attention", "mixer": dict(
        {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "mask": {"size": win}, "scale": scale}, **({"kv_from": src} if src is not None else {}))}
    moe = lambda E, top, ff, lim, sc: {"kind": "moe", "router": {"experts": E, "top": top, "scale": sc}, "expert": {"ff": ff, "limit": lim}}
    layers = [dict(att(3, 12, 20, 40, 7, 0.3), mlp=moe(5, 2, 24, 1.5, 1.25)),
              dict(ssd(6, 10, 12, 3, 3, 2), mlp=None),
              dict(att(5, 8, 8, 40, 19, 0.25, 0), mlp=moe(7, 1, 16, 3.0, 0.75)),
              dict(ssd(4, 8, 24, 1, 4, 1), mlp=moe(4, 3, 20, 2.5, 1.0)),
              dict(att(2, 16, 12, 24, 5, 0.2), mlp=None)]
    layers[3]["type"] = "mamba2_2"
    cfg = {"architecture": "Desarax", "vocab": 61, "width": 48, "layers": layers, "norm": {"eps": 1e-5, "groups": 3},
           "residual_mult": 0.7, "logit_scale": 1.5, "token_side": {"dim": 6}}
    cfg.update(kw)
    return cfg
