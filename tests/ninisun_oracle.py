"""Plain float64 restatement of the Ninisun design, one function per mechanism, written from its equations.

Slow on purpose (python loops over keys and tokens) and shares no code with the served path: the tests compare the
engine's kernels, cache, state slots and scheduler with these functions.  Weights are a dict name -> tensor in the
checkpoint's own names; the config is the checkpoint's config.json as a dict.

Notation: h = a sublayer's input row, H query heads over G key/value heads (query head n reads key/value head
n // (H // G)), positions count from 0 in every sequence.
"""
import math

import torch

F64 = torch.float64


def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis."""
    x = x.to(F64)
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w.to(F64)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def sigmoid(z):
    return 1.0 / (1.0 + torch.exp(-z))


def rotary_table(rot, positions):
    """cos, sin [len(positions), dims / 2] for the rotation config `rot` (base, dims, optional scaling)."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=F64)
    f = base ** (-2.0 * i / dims)
    mag = 1.0
    sc = rot.get("scaling")
    if sc:
        factor, orig = float(sc["factor"]), float(sc["original"])

        def turn_dim(t):
            return dims * math.log(orig / (2.0 * math.pi * t)) / (2.0 * math.log(base))

        lo = max(math.floor(turn_dim(float(sc["fast"]))), 0)
        hi = min(math.ceil(turn_dim(float(sc["slow"]))), dims - 1)
        ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        f = f / factor * ramp + f * (1.0 - ramp)
        mag = 0.1 * math.log(factor) + 1.0
    ang = torch.as_tensor(positions, dtype=F64)[:, None] * f[None, :]
    return torch.cos(ang) * mag, torch.sin(ang) * mag


def rotate_pairs(x, cos, sin):
    """x [tokens, heads, dim]: the first 2 * cos.shape[1] columns of every head are rotated as pairs (2i, 2i + 1)."""
    x = x.to(F64).clone()
    n = cos.shape[1]
    a, b = x[..., 0:2 * n:2].clone(), x[..., 1:2 * n:2].clone()
    c, s = cos[:, None, :], sin[:, None, :]
    x[..., 0:2 * n:2] = a * c - b * s
    x[..., 1:2 * n:2] = b * c + a * s
    return x


def visible(T, size, keep_first):
    """[T, T] matrix: key j is visible to query i when j <= i and (i - j < size or j < keep_first); size <= 0: all j <= i."""
    vis = torch.zeros(T, T, dtype=torch.bool)
    for i in range(T):
        for j in range(i + 1):
            vis[i, j] = size <= 0 or i - j < size or j < keep_first
    return vis


def window_softmax_attention(q, k, v, scale, size, keep_first):
    """q [T, H, d], k [T, G, d], v [T, G, e] of ONE sequence from position 0; softmax over the visible keys."""
    T, H, _ = q.shape
    G = k.shape[1]
    vis = visible(T, size, keep_first)
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for n in range(H):
        g = n // (H // G)
        s = (q[:, n] @ k[:, g].T) * scale
        p = torch.softmax(s.masked_fill(~vis, -math.inf), -1)
        out[:, n] = p @ v[:, g]
    return out


def causal_sigmoid_attention(q, k, v, scale, head_bias):
    """Unnormalised weights sigmoid(score + head_bias[n]) over every j <= i."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for n in range(H):
        g = n // (H // G)
        s = (q[:, n] @ k[:, g].T) * scale + head_bias[n]
        w = torch.tril(sigmoid(s))
        out[:, n] = w @ v[:, g]
    return out


def delta_rule(r, k, v, w, a, state=None):
    """Generalised delta rule of one sequence.  r, k, v, w, a: [T, heads, d].  With u = k / sqrt(sum k^2 + 1e-6):
    S <- diag(w) S - (a * u) (u^T S) + k v^T (both first terms read the old S), o = S^T r.  Returns o, final S."""
    T, N, d = r.shape
    S = torch.zeros(N, d, d, dtype=F64) if state is None else state.clone()
    o = torch.zeros(T, N, d, dtype=F64)
    for t in range(T):
        for n in range(N):
            kk = k[t, n]
            u = kk / torch.sqrt((kk * kk).sum() + 1e-6)
            old = S[n]
            S[n] = w[t, n][:, None] * old - (a[t, n] * u)[:, None] * (u @ old)[None, :] + kk[:, None] * v[t, n][None, :]
            o[t, n] = S[n].T @ r[t, n]
    return o, S


def lin(W, x, b=None):
    y = x.to(F64) @ W.to(F64).T
    return y if b is None else y + b.to(F64)


def attention_mixer(p, m, Wt, h, positions, v_first, is_first):
    """Mixer 'attention' on one whole sequence.  Returns (output, the values that later v_mix layers mix in)."""
    T = h.shape[0]
    H, G, d, e = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m.get("vdim", m["dim"])
    q = lin(Wt[p + "q"], h).view(T, H, d)
    k = lin(Wt[p + "k"], h).view(T, G, d)
    v = lin(Wt[p + "v"], h).view(T, G, e)
    rot = m.get("rot")
    if rot:
        cos, sin = rotary_table(rot, positions)
        q, k = rotate_pairs(q, cos, sin), rotate_pairs(k, cos, sin)
    if m.get("v_mix"):
        if is_first:
            v_first = v
        else:
            lam = Wt[p + "vmix"].to(F64)
            v = (1.0 - lam) * v + lam * v_first
    mask = m.get("mask") or {}
    o = window_softmax_attention(q, k, v, float(m["scale"]), int(mask.get("size", 0) or 0), int(mask.get("keep_first", 0) or 0))
    return lin(Wt[p + "o"], o.reshape(T, H * e)), v_first


def parallel_mixer(p, m, Wt, h, positions, eps):
    """Mixer 'parallel': gated sigmoid attention beside a delta-rule recurrence, both reading h."""
    T = h.shape[0]
    L, R = m["left"], m["right"]
    H, G, d, e = L["heads"], L.get("kv_heads", L["heads"]), L["dim"], L.get("vdim", L["dim"])
    lp = p + "left."
    q = lin(Wt[lp + "q"], h, Wt[lp + "q.b"]).view(T, H, d)
    k = lin(Wt[lp + "k"], h, Wt[lp + "k.b"]).view(T, G, d)
    v = lin(Wt[lp + "v"], h, Wt[lp + "v.b"]).view(T, G, e)
    rot = L.get("rot")
    if rot:
        cos, sin = rotary_table(rot, positions)
        q, k = rotate_pairs(q, cos, sin), rotate_pairs(k, cos, sin)
    o = causal_sigmoid_attention(q, k, v, float(L["scale"]), Wt[lp + "pb"].to(F64))
    o = o * sigmoid(lin(Wt[lp + "g"], h))[:, :, None]
    left = lin(Wt[lp + "o"], o.reshape(T, H * e))
    N, dr = R["heads"], R["dim"]
    rp = p + "right."
    r = lin(Wt[rp + "r"], h).view(T, N, dr)
    kk = lin(Wt[rp + "k"], h).view(T, N, dr)
    vv = lin(Wt[rp + "v"], h).view(T, N, dr)
    dec = lin(Wt[rp + "w2"], torch.tanh(lin(Wt[rp + "w1"], h))) + Wt[rp + "w0"].to(F64)
    w = torch.exp(-math.exp(-0.5) * sigmoid(dec)).view(T, N, dr)
    a = sigmoid(lin(Wt[rp + "a"], h, Wt[rp + "a.b"])).view(T, N, dr)
    ro, _ = delta_rule(r, kk, vv, w, a)
    ro = rms_norm(ro, None, eps).reshape(T, N * dr) * Wt[rp + "norm"].to(F64) * sigmoid(lin(Wt[rp + "g"], h))
    right = lin(Wt[rp + "o"], ro)
    return float(m["left_scale"]) * left + float(m["right_scale"]) * right


def feed_forward(p, ml, Wt, h):
    if ml["kind"] != "dense":
        raise ValueError(ml["kind"])
    return lin(Wt[p + "down"], gelu_tanh(lin(Wt[p + "gate"], h)) * lin(Wt[p + "up"], h))


def forward(cfg, Wt, tokens, layer_sink=None):
    """Logits [T, vocab] (float64) of one whole sequence from position 0."""
    eps = float(cfg["norm"]["eps"])
    T = len(tokens)
    positions = list(range(T))
    x = Wt["embed"].to(F64)[torch.as_tensor(tokens, dtype=torch.long)]
    v_first, seen_vmix = None, False
    for i, L in enumerate(cfg["layers"]):
        p = "l%d." % i
        h = rms_norm(x, Wt[p + "norm1"], eps)
        if L["type"] == "attention":
            vm = bool(L["mixer"].get("v_mix"))
            y, v_first = attention_mixer(p + "mix.", L["mixer"], Wt, h, positions, v_first, vm and not seen_vmix)
            seen_vmix = seen_vmix or vm
        elif L["type"] == "parallel":
            y = parallel_mixer(p + "mix.", L["mixer"], Wt, h, positions, eps)
        else:
            raise ValueError(L["type"])
        x = x + rms_norm(y, Wt[p + "norm1b"], eps) * Wt[p + "ls1"].to(F64)
        if L.get("mlp"):
            y = feed_forward(p + "mlp.", L["mlp"], Wt, rms_norm(x, Wt[p + "norm2"], eps))
            x = x + rms_norm(y, Wt[p + "norm2b"], eps) * Wt[p + "ls2"].to(F64)
        if layer_sink is not None:
            layer_sink.append(x.clone())
    return lin(Wt["embed"], rms_norm(x, Wt["final.norm"], eps))


# ------------------------------------------------------------------ random checkpoints
def make_config(vocab=96, width=48, eps=1e-5, layers=None):
    return {"architecture": "Ninisun", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


def rot(dims, base=10000.0, scaling=None):
    r = {"dims": dims, "base": base}
    if scaling:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


def attn(heads=4, kv_heads=2, dim=8, vdim=16, scale=0.3, rot_dims=4, base=10000.0, window=24, keep_first=2, v_mix=True):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot_dims:
        m["rot"] = rot(rot_dims, base)
    if window:
        m["mask"] = {"size": window, "keep_first": keep_first}
    if v_mix:
        m["v_mix"] = True
    return m


def parallel(heads=4, kv_heads=2, dim=8, vdim=16, scale=0.25, rot_dims=8, base=5000.0, scaling=(4.0, 64, 16.0, 1.0),
             r_heads=3, r_dim=8, left_scale=0.7, right_scale=1.3):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot_dims:
        left["rot"] = rot(rot_dims, base, scaling)
    return {"left": left, "right": {"heads": r_heads, "dim": r_dim}, "left_scale": left_scale, "right_scale": right_scale}


def layer(mixer, ff=40):
    return {"type": "parallel" if "left" in mixer else "attention", "mixer": mixer,
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def make_checkpoint(cfg, seed=0, dtype=torch.bfloat16, lora=6):
    """Random tensors under the checkpoint's names, rounded to `dtype` (engine and oracle then see the same numbers)."""
    g = torch.Generator().manual_seed(seed)
    D = cfg["width"]
    T = {}

    def lin(name, out, inp, gain=1.0):
        T[name] = (torch.randn(out, inp, generator=g) * gain / math.sqrt(inp)).to(dtype)

    def vec(name, n, mean=1.0, std=0.1):
        T[name] = (mean + std * torch.randn(n, generator=g)).to(dtype)

    T["embed"] = torch.randn(cfg["vocab"], D, generator=g).to(dtype)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        for n in ("norm1", "norm1b"):
            vec(p + n, D)
        vec(p + "ls1", D, 0.5, 0.2)
        if L["type"] == "attention":
            H, G, d, e = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m.get("vdim", m["dim"])
            lin(p + "mix.q", H * d, D, 2.0), lin(p + "mix.k", G * d, D, 2.0), lin(p + "mix.v", G * e, D), lin(p + "mix.o", D, H * e)
            if m.get("v_mix"):
                T[p + "mix.vmix"] = (0.2 + 0.6 * torch.rand((), generator=g)).to(dtype)
        else:
            l, r = m["left"], m["right"]
            H, G, d, e = l["heads"], l.get("kv_heads", l["heads"]), l["dim"], l.get("vdim", l["dim"])
            q = p + "mix.left."
            lin(q + "q", H * d, D, 2.0), lin(q + "k", G * d, D, 2.0), lin(q + "v", G * e, D), lin(q + "o", D, H * e, 0.3)
            vec(q + "q.b", H * d, 0.0, 0.3), vec(q + "k.b", G * d, 0.0, 0.3), vec(q + "v.b", G * e, 0.0, 0.3)
            vec(q + "pb", H, -1.0, 1.0), lin(q + "g", H, D, 2.0)
            nd, q = r["heads"] * r["dim"], p + "mix.right."
            for n in ("r", "k", "v"):
                lin(q + n, nd, D)
            lin(q + "g", nd, D, 2.0), lin(q + "a", nd, D, 2.0), vec(q + "a.b", nd, 0.0, 0.5)
            lin(q + "w1", lora, D, 2.0), lin(q + "w2", nd, lora, 2.0), vec(q + "w0", nd, 0.0, 1.0)
            vec(q + "norm", nd), lin(q + "o", D, nd)
        if L.get("mlp"):
            ff = L["mlp"]["ff"]
            for n in ("norm2", "norm2b"):
                vec(p + n, D)
            vec(p + "ls2", D, 0.5, 0.2)
            lin(p + "mlp.gate", ff, D), lin(p + "mlp.up", ff, D), lin(p + "mlp.down", D, ff)
    vec("final.norm", D)
    return T
