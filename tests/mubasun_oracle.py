"""Plain, slow restatement of the Mubasun design on the CPU (float64), one function per mechanism, written from the
design's equations.  It shares no code with the engine: tensors are looked up by checkpoint name, attention loops over
queries, experts loop over tokens.  `make_checkpoint` draws random weights for a configuration dictionary."""
import math

import torch

F64 = torch.float64


# ------------------------------------------------------------------ mechanisms
def group_rms_norm(x, w, groups, eps):
    """Split the last axis into `groups` equal consecutive parts, divide each by sqrt(mean(part^2) + eps), times w."""
    out = torch.empty_like(x)
    size = x.shape[-1] // groups
    for g in range(groups):
        part = x[..., g * size:(g + 1) * size]
        out[..., g * size:(g + 1) * size] = part / torch.sqrt((part * part).mean(-1, keepdim=True) + eps)
    return out * w


def whole_rms_norm(x, w, eps):
    """RMS norm over the whole projection row (all heads at once), plain weight."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def head_slopes(heads):
    return [2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)]


def window_attention(q, k_cache, v_cache, positions, heads, kv_heads, dim, vdim, scale, window):
    """q: [n, heads*dim] for queries at `positions`; k_cache / v_cache: [len, kv_heads*dim|vdim] of the sequence.
    Query at i sees j with 0 <= i - j < window (window 0: every j <= i)."""
    out = torch.zeros(q.shape[0], heads * vdim, dtype=q.dtype)
    slopes = head_slopes(heads)
    for r, i in enumerate(positions):
        lo = 0 if window <= 0 else max(0, i - window + 1)
        back = torch.arange(i - lo, -1, -1, dtype=q.dtype)            # i - j for j = lo .. i
        for h in range(heads):
            g = h // (heads // kv_heads)
            qh = q[r, h * dim:(h + 1) * dim]
            s = (k_cache[lo:i + 1, g * dim:(g + 1) * dim] @ qh) * scale - slopes[h] * back
            out[r, h * vdim:(h + 1) * vdim] = torch.softmax(s, 0) @ v_cache[lo:i + 1, g * vdim:(g + 1) * vdim]
    return out


def xielu(z, p, q):
    sp, sq = math.log1p(math.exp(p)), math.log1p(math.exp(q))
    pos = sp * z * z + z / 2
    neg = (0.5 + sq) * (torch.exp(z) - 1 - z) + z / 2
    return torch.where(z > 0, pos, neg)


def silu(z):
    return z * torch.sigmoid(z)


def route(h, w_router, correction, top, scale):
    """-> (indices [n, top], weights [n, top]); choice by score + correction, weight = score * scale."""
    s = torch.softmax(h @ w_router.t(), -1)
    choice = s + correction if correction is not None else s
    idx = torch.argsort(choice, dim=-1, descending=True, stable=True)[:, :top]
    return idx, torch.gather(s, 1, idx) * scale


def gated_expert(h, w_gate, w_up, w_down):
    return (silu(h @ w_gate.t()) * (h @ w_up.t())) @ w_down.t()


def moe_ff(h, W, prefix, ml):
    r = ml["router"]
    E, I = r["experts"], r.get("identity", 0)
    idx, wts = route(h, W[prefix + "router"], W.get(prefix + "correction"), r["top"], r.get("scale", 1.0))
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, w in zip(idx[t].tolist(), wts[t]):
            if e < E:
                p = f"{prefix}e{e}."
                out[t] += w * gated_expert(h[t:t + 1], W[p + "gate"], W[p + "up"], W[p + "down"])[0]
            else:
                assert e < E + I
                out[t] += w * h[t]
    if ml.get("shared"):
        p = prefix + "shared."
        out = out + gated_expert(h, W[p + "gate"], W[p + "up"], W[p + "down"]) * torch.sigmoid(h @ W[p + "sg"].t())
    return out


def dense_ff(h, W, prefix):
    return xielu(h @ W[prefix + "up"].t(), float(W[prefix + "act"][0]), float(W[prefix + "act"][1])) @ W[prefix + "down"].t()


# ------------------------------------------------------------------ the model
class Oracle:
    """Holds float64 weights and a per-sequence cache of keys / values, so that a prompt can be run whole, in
    portions, or token by token with the same functions."""

    def __init__(self, cfg, tensors):
        self.cfg = cfg
        self.W = {k: v.to(F64) for k, v in tensors.items()}

    def new_cache(self):
        return {i: (torch.zeros(0, 0, dtype=F64), torch.zeros(0, 0, dtype=F64)) for i in range(len(self.cfg["layers"]))}

    def run(self, tokens, cache, start, layers_out=None):
        """tokens at positions start .. start+n-1 of the sequence that owns `cache`; returns logits [n, vocab]."""
        cfg, W = self.cfg, self.W
        eps, groups = cfg["norm"]["eps"], cfg["norm"]["groups"]
        n = len(tokens)
        positions = list(range(start, start + n))
        x = W["embed"][tokens] + W["pos"][positions]
        for li, L in enumerate(cfg["layers"]):
            p, m = f"l{li}.", L["mixer"]
            H, G, dim = m["heads"], m.get("kv_heads", m["heads"]), m["dim"]
            vdim = m.get("vdim", dim)
            h = group_rms_norm(x, W[p + "norm1"], groups, eps)
            q = whole_rms_norm(h @ W[p + "mix.q"].t(), W[p + "mix.q.norm"], eps)
            if m.get("kv_from") is None:
                k = whole_rms_norm(h @ W[p + "mix.k"].t(), W[p + "mix.k.norm"], eps)
                v = h @ W[p + "mix.v"].t()
                ck, cv = cache[li]
                ck = torch.cat([ck.reshape(-1, G * dim), k], 0)
                cv = torch.cat([cv.reshape(-1, G * vdim), v], 0)
                cache[li] = (ck, cv)
            else:
                ck, cv = cache[m["kv_from"]]
            window = (m.get("mask") or {}).get("size", 0)
            o = window_attention(q, ck, cv, positions, H, G, dim, vdim, m["scale"], window)
            o = o * torch.sigmoid(h @ W[p + "mix.g"].t())
            y = o @ W[p + "mix.o"].t()
            ml = L.get("mlp")
            if ml is not None:
                y = y + (dense_ff(h, W, p + "mlp.") if ml["kind"] == "dense" else moe_ff(h, W, p + "mlp.", ml))
            x = x + y
            if layers_out is not None:
                layers_out.append(x.clone())
        return group_rms_norm(x, W["final.norm"], groups, eps) @ W["head"].t()

    def logits(self, tokens):
        return self.run(list(tokens), self.new_cache(), 0)

    def greedy(self, prompt, n_new):
        cache = self.new_cache()
        lg = self.run(list(prompt), cache, 0)
        out, pos = [], len(prompt)
        for _ in range(n_new):
            out.append(int(torch.argmax(lg[-1])))
            lg = self.run([out[-1]], cache, pos)
            pos += 1
        return out


# ------------------------------------------------------------------ random checkpoints
def make_config(vocab=96, width=48, max_positions=256, groups=3, eps=1e-5, layers=None):
    return {"architecture": "Mubasun", "vocab": vocab, "width": width, "max_positions": max_positions,
            "norm": {"eps": eps, "groups": groups}, "layers": layers}


def attn(heads=4, kv_heads=2, dim=8, vdim=16, window=24, scale=0.3, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def layer(mixer, mlp):
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def moe(experts=5, identity=1, top=2, ff=24, scale=1.5, shared=16):
    d = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top, "scale": scale}}
    if shared:
        d["shared"] = {"ff": shared}
    return d


def make_checkpoint(cfg, seed=0, dtype=torch.bfloat16):
    """Random tensors under the checkpoint's names, rounded to `dtype` (the engine and the oracle then see the
    same numbers)."""
    g = torch.Generator().manual_seed(seed)
    D = cfg["width"]
    T = {}

    def lin(name, out, inp, gain=1.0):
        T[name] = (torch.randn(out, inp, generator=g) * gain / math.sqrt(inp)).to(dtype)

    def vec(name, n, mean=1.0, std=0.1):
        T[name] = (mean + std * torch.randn(n, generator=g)).to(dtype)

    T["embed"] = torch.randn(cfg["vocab"], D, generator=g).to(dtype)
    T["pos"] = (0.5 * torch.randn(cfg["max_positions"], D, generator=g)).to(dtype)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        H, G, dim = m["heads"], m.get("kv_heads", m["heads"]), m["dim"]
        vdim = m.get("vdim", dim)
        vec(p + "norm1", D)
        lin(p + "mix.q", H * dim, D)
        vec(p + "mix.q.norm", H * dim, 1.0, 0.3)
        if m.get("kv_from") is None:
            lin(p + "mix.k", G * dim, D)
            lin(p + "mix.v", G * vdim, D)
            vec(p + "mix.k.norm", G * dim, 1.0, 0.3)
        lin(p + "mix.g", H * vdim, D, 2.0)
        lin(p + "mix.o", D, H * vdim)
        ml = L.get("mlp")
        if ml is None:
            continue
        if ml["kind"] == "dense":
            lin(p + "mlp.up", ml["ff"], D)
            lin(p + "mlp.down", D, ml["ff"])
            T[p + "mlp.act"] = torch.randn(2, generator=g).to(dtype)
        else:
            r = ml["router"]
            for e in range(r["experts"]):
                lin(f"{p}mlp.e{e}.gate", ml["expert"]["ff"], D)
                lin(f"{p}mlp.e{e}.up", ml["expert"]["ff"], D)
                lin(f"{p}mlp.e{e}.down", D, ml["expert"]["ff"])
            n_route = r["experts"] + r.get("identity", 0)
            lin(p + "mlp.router", n_route, D, 3.0)
            vec(p + "mlp.correction", n_route, 0.0, 0.2)
            if ml.get("shared"):
                s = p + "mlp.shared."
                lin(s + "gate", ml["shared"]["ff"], D)
                lin(s + "up", ml["shared"]["ff"], D)
                lin(s + "down", D, ml["shared"]["ff"])
                lin(s + "sg", 1, D, 2.0)
    vec("final.norm", D)
    lin("head", cfg["vocab"], D)
    return T
