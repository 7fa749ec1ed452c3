"""Plain, slow restatement of the Gufotar design for the tests: one function per mechanism, token loops where the
definition is a recurrence, float64 by default. It shares no code with ``lite_llama_b200``.

A model is ``(cfg, w)``: ``cfg`` the dictionary a ``config.json`` of this design holds, ``w`` a name -> tensor map
with the checkpoint's tensor names. Linear weights are ``[out, in]``.
"""

from __future__ import annotations

import math

import torch


# ------------------------------------------------------------------ pieces #
def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last dimension."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def zero_centred_norm(x, weight, eps):
    """RMS norm whose stored weight is an offset from one."""
    return rms_unit(x, eps) * (1.0 + weight)


def silu(z):
    return z / (1.0 + torch.exp(-z))


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def causal_conv(u, taps_w, bias, history=None):
    """Per-channel causal convolution over time. ``u [T, C]``, ``taps_w [C, K]`` (last column multiplies the current
    token), ``history [K-1, C]`` = the inputs before ``u`` (zeros at a sequence start). Returns (out, new history)."""
    T, C = u.shape
    K = taps_w.shape[1]
    if history is None:
        history = u.new_zeros(K - 1, C)
    ext = torch.cat([history, u], 0)
    out = u.new_zeros(T, C)
    for t in range(T):
        window = ext[t:t + K]                          # [K, C], oldest first
        out[t] = (window * taps_w.t()).sum(0) + bias
    return out, ext[ext.shape[0] - (K - 1):].clone()


def ssm_recurrence(x, dt, a_log, b, c, d_skip, state=None):
    """State-space recurrence of one sequence, token by token.
    ``x [T, H, P]``, ``dt [T, H]`` (already positive), ``b, c [T, G, N]``; head h reads group h // (H // G).
    S_t = exp(-exp(a_log) dt_t) S_{t-1} + dt_t b_t x_t^T  (S: [H, N, P]);  y_t = S_t^T c_t + d x_t."""
    T, H, P = x.shape
    G, N = b.shape[1], b.shape[2]
    per = H // G
    if state is None:
        state = x.new_zeros(H, N, P)
    state = state.clone()
    y = x.new_zeros(T, H, P)
    for t in range(T):
        for h in range(H):
            g = h // per
            decay = torch.exp(-torch.exp(a_log[h]) * dt[t, h])
            state[h] = decay * state[h] + dt[t, h] * torch.outer(b[t, g], x[t, h])
            y[t, h] = state[h].t() @ c[t, g] + d_skip[h] * x[t, h]
    return y, state


def grouped_gated_norm(y, z, weight, groups, eps):
    """Gate first, then unit RMS in ``groups`` equal parts of the last dimension, then the weight."""
    g = y * silu(z)
    T, inner = g.shape
    parts = g.view(T, groups, inner // groups)
    return rms_unit(parts, eps).reshape(T, inner) * weight


def mamba2_mixer(h, w, pre, m, eps, carry=None):
    """``h [T, width]`` of ONE sequence; ``carry`` = (conv history, state) from its earlier tokens."""
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    proj = h @ w[pre + "in"].t()
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    hist, state = carry if carry is not None else (None, None)
    conv, hist = causal_conv(xbc, w[pre + "conv"], w[pre + "conv.b"], hist)
    conv = silu(conv)
    x = conv[:, :inner].reshape(-1, H, P)
    b = conv[:, inner:inner + G * N].reshape(-1, G, N)
    c = conv[:, inner + G * N:].reshape(-1, G, N)
    dt = softplus(dt + w[pre + "dt_bias"])
    y, state = ssm_recurrence(x, dt, w[pre + "A_log"], b, c, w[pre + "D"], state)
    y = grouped_gated_norm(y.reshape(-1, inner), z, w[pre + "norm"], m["norm_groups"], eps)
    return y @ w[pre + "o"].t(), (hist, state)


def query_temperature(positions, q_temp):
    if not q_temp:
        return torch.ones_like(positions, dtype=torch.float64)
    steps = torch.floor((positions.double() + 1.0) / q_temp["every"])
    return 1.0 + q_temp["coef"] * torch.log(steps + 1.0)


def sink_attention(q, k, v, q_pos, k_pos, scale, softcap, sink):
    """``q [Tq, H, D]``, ``k [Tk, G, D]``, ``v [Tk, G, Dv]``; query at position p sees keys at positions <= p.
    The sink adds exp(sink_h) to the softmax denominator and nothing to the numerator."""
    Tq, H, _ = q.shape
    G = k.shape[1]
    per = H // G
    out = q.new_zeros(Tq, H, v.shape[2])
    for i in range(Tq):
        seen = k_pos <= q_pos[i]
        for h in range(H):
            g = h // per
            s = (k[seen, g] @ q[i, h]) * scale
            if softcap:
                s = softcap * torch.tanh(s / softcap)
            top = s.max()
            if sink is not None:
                top = torch.maximum(top, sink[h])
            e = torch.exp(s - top)
            den = e.sum()
            if sink is not None:
                den = den + torch.exp(sink[h] - top)
            out[i, h] = (e / den) @ v[seen, g]
    return out


def attention_mixer(h, positions, w, pre, m, eps, v_first, kv_carry=None):
    """One sequence. ``v_first``: None in the first value-mixing layer (its values are returned for the later ones),
    else that layer's values of these tokens. ``kv_carry`` = (k, v, positions) of the sequence's earlier tokens."""
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_unit(h @ w[pre + "q"].t(), eps) * w[pre + "q.norm"]        # over the whole projection, plain weight
    k = rms_unit(h @ w[pre + "k"].t(), eps) * w[pre + "k.norm"]
    v = h @ w[pre + "v"].t()
    v_own = v
    if m.get("v_mix") and v_first is not None:
        lam = w[pre + "vmix"]
        v = (1.0 - lam) * v + lam * v_first
    q = q * query_temperature(positions, m.get("q_temp")).to(q.dtype)[:, None]
    q, k, v = q.view(-1, H, D), k.view(-1, G, D), v.reshape(-1, G, Dv)
    k_all, v_all, p_all = k, v, positions
    if kv_carry is not None:
        k_all, v_all, p_all = torch.cat([kv_carry[0], k]), torch.cat([kv_carry[1], v]), torch.cat([kv_carry[2], positions])
    sink = w.get(pre + "sink")
    o = sink_attention(q, k_all, v_all, positions, p_all, m["scale"], m.get("softcap"), sink)
    return o.reshape(-1, H * Dv) @ w[pre + "o"].t(), v_own, (k_all, v_all, p_all)


def dense_ff(h, w, pre):
    return (torch.relu(h @ w[pre + "up"].t()) ** 2) @ w[pre + "down"].t()


# ------------------------------------------------------------------- model #
class Oracle:
    """Runs sequences one at a time and keeps what each has seen, so a sequence may be fed in portions."""

    def __init__(self, cfg: dict, weights: dict, dtype=torch.float64):
        self.cfg = cfg
        self.w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
        self.dtype = dtype
        self.carry: dict = {}

    def forward(self, tokens, seq="s", keep_layers=False):
        cfg, w, eps = self.cfg, self.w, self.cfg["norm"]["eps"]
        st = self.carry.setdefault(seq, {"n": 0, "layers": {}})
        start = st["n"]
        positions = torch.arange(start, start + len(tokens))
        x = w["embed"][torch.as_tensor(tokens)] + w["pos"][positions]
        v_first, trace = None, []
        for i, layer in enumerate(cfg["layers"]):
            pre = f"l{i}.mix."
            if layer["type"] == "mamba2":
                y, st["layers"][i] = mamba2_mixer(x, w, pre, layer["mixer"], eps, st["layers"].get(i))
            elif layer["type"] == "attention":
                share = v_first if layer["mixer"].get("v_mix") else None
                y, v_own, st["layers"][i] = attention_mixer(x, positions, w, pre, layer["mixer"], eps, share,
                                                            st["layers"].get(i))
                if layer["mixer"].get("v_mix") and v_first is None:
                    v_first = v_own
            else:
                raise ValueError(layer["type"])
            x = x + zero_centred_norm(y, w[f"l{i}.norm1"], eps)
            if layer.get("mlp"):
                x = x + zero_centred_norm(dense_ff(x, w, f"l{i}.mlp."), w[f"l{i}.norm2"], eps)
            if keep_layers:
                trace.append(x.clone())
        st["n"] = start + len(tokens)
        logits = zero_centred_norm(x, w["final.norm"], eps) @ w["head"].t()
        return (logits, torch.stack(trace)) if keep_layers else logits

    def drop(self, seq="s"):
        self.carry.pop(seq, None)


# -------------------------------------------------------- random instances #
def random_model(cfg: dict, seed: int = 0, spread: float = 1.0):
    """Random bfloat16-representable weights with the checkpoint's names and shapes."""
    g = torch.Generator().manual_seed(seed)
    width = cfg["width"]

    def mat(o, i, s=1.0):
        return (torch.randn(o, i, generator=g) * s * spread / math.sqrt(i)).bfloat16().float()

    def vec(n, s=0.2, shift=0.0):
        return (torch.randn(n, generator=g) * s + shift).bfloat16().float()

    w = {}
    w["embed"] = (torch.randn(cfg["vocab"], width, generator=g)).bfloat16().float()
    w["pos"] = (torch.randn(cfg["max_positions"], width, generator=g) * 0.3).bfloat16().float()
    for i, layer in enumerate(cfg["layers"]):
        m, pre = layer["mixer"], f"l{i}.mix."
        w[f"l{i}.norm1"] = vec(width)
        if layer["type"] == "mamba2":
            inner, gn = m["heads"] * m["vdim"], m["groups"] * m["state"]
            w[pre + "in"] = mat(2 * inner + 2 * gn + m["heads"], width)
            w[pre + "conv"] = (torch.randn(inner + 2 * gn, m["conv"], generator=g) * 0.5).bfloat16().float()
            w[pre + "conv.b"] = vec(inner + 2 * gn)
            w[pre + "dt_bias"] = vec(m["heads"], 0.5, -1.0)
            w[pre + "A_log"] = vec(m["heads"], 0.5, -1.0)
            w[pre + "D"] = vec(m["heads"], 0.5, 1.0)
            w[pre + "norm"] = vec(inner, 0.2, 1.0)
            w[pre + "o"] = mat(width, inner)
        else:
            w[pre + "q"] = mat(m["heads"] * m["dim"], width)
            w[pre + "k"] = mat(m["kv_heads"] * m["dim"], width)
            w[pre + "v"] = mat(m["kv_heads"] * m["vdim"], width)
            w[pre + "q.norm"] = vec(m["heads"] * m["dim"], 0.4, 1.2)
            w[pre + "k.norm"] = vec(m["kv_heads"] * m["dim"], 0.4, 1.2)
            w[pre + "vmix"] = vec(1, 0.1, 0.4).reshape(())
            w[pre + "sink"] = vec(m["heads"], 1.0)
            w[pre + "o"] = mat(width, m["heads"] * m["vdim"])
        if layer.get("mlp"):
            w[f"l{i}.norm2"] = vec(width)
            w[f"l{i}.mlp.up"] = mat(layer["mlp"]["ff"], width)
            w[f"l{i}.mlp.down"] = mat(width, layer["mlp"]["ff"])
    w["final.norm"] = vec(width)
    w["head"] = mat(cfg["vocab"], width)
    return w


def attention_layer(heads=4, kv_heads=2, dim=16, vdim=24, scale=0.3, softcap=8.0, v_mix=True, coef=0.25, every=5,
                    ff=48):
    mixer = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "scale": scale, "softcap": softcap, "v_mix": v_mix,
             "vdim": vdim, "q_temp": {"coef": coef, "every": every}}
    return {"type": "attention", "mixer": mixer, "mlp": {"ff": ff, "kind": "dense"} if ff else None}


def mamba2_layer(heads=6, vdim=8, state=12, groups=2, norm_groups=3, conv=3, ff=0):
    mixer = {"conv": conv, "groups": groups, "heads": heads, "norm_groups": norm_groups, "state": state, "vdim": vdim}
    return {"type": "mamba2", "mixer": mixer, "mlp": {"ff": ff, "kind": "dense"} if ff else None}


def make_config(layers, width=40, vocab=96, max_positions=256, eps=1e-5):
    return {"architecture": "Gufotar", "layers": layers, "max_positions": max_positions, "norm": {"eps": eps},
            "vocab": vocab, "width": width}
