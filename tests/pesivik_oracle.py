"""Plain float64 restatement of the Pesivik design, one function per mechanism, token loops instead of batched
kernels.  Shares no code with the package: the tests compare the CUDA path with this.

A model is ``(config, tensors)``: ``config`` is the dict form of ``config.json`` (keys ``width``, ``vocab``,
``embedding.scale``, ``norm.eps``, ``logit_softcap``, ``layers``), ``tensors`` maps checkpoint names to arrays.
"""

from __future__ import annotations

import math

import numpy as np


def f64(t) -> np.ndarray:
    if hasattr(t, "detach"):
        t = t.detach().cpu().double().numpy()
    return np.asarray(t, dtype=np.float64)


# ------------------------------------------------------------------------------------------------- small pieces #
def rms_unit(x: np.ndarray, eps: float) -> np.ndarray:
    return x / math.sqrt(float(np.mean(x * x)) + eps)


def rms_norm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    return rms_unit(x, eps) * w


def layer_norm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    mu = float(np.mean(x))
    var = float(np.mean((x - mu) ** 2))
    return (x - mu) / math.sqrt(var + eps) * w


def gelu_erf(z: np.ndarray) -> np.ndarray:
    return np.array([0.5 * v * (1.0 + math.erf(v / math.sqrt(2.0))) for v in z.ravel()]).reshape(z.shape)


def sigmoid(z: np.ndarray) -> np.ndarray:
    return 1.0 / (1.0 + np.exp(-z))


def rotate(vec: np.ndarray, pos: int, dims: int, base: float) -> np.ndarray:
    """Rotate-half layout on the first ``dims`` entries: entry i pairs with entry i + dims/2; the rest is untouched."""
    out = vec.copy()
    half = dims // 2
    for i in range(half):
        a = pos * base ** (-2.0 * i / dims)
        u, v = vec[i], vec[i + half]
        out[i] = u * math.cos(a) - v * math.sin(a)
        out[i + half] = v * math.cos(a) + u * math.sin(a)
    return out


def soft_cap(logits: np.ndarray, cap: float) -> np.ndarray:
    return cap * np.tanh(logits / cap) if cap else logits


# ------------------------------------------------------------------------------------------------ the mixer #
def latent_attention(h: np.ndarray, positions: list[int], m: dict, w: dict, eps: float) -> np.ndarray:
    """``h [T, width]`` = one whole sequence (normed mixer input); returns ``[T, width]``.  Keys and values are
    expanded from the latent for every token (the direct form), each query walks its window."""
    H, dim, rot, vdim, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    rdims, base, window, scale = m["rot"]["dims"], float(m["rot"]["base"]), m["mask"]["size"], float(m["scale"])
    T = h.shape[0]
    q_all, k_all, v_all, kr_all, gate_all = [], [], [], [], []
    for t in range(T):
        cq = rms_norm(w["dq"] @ h[t], w["dq.norm"], eps)
        q = (w["uq"] @ cq).reshape(H, dim + rot)
        q = np.stack([np.concatenate([q[i, :dim], rotate(q[i, dim:], positions[t], rdims, base)]) for i in range(H)])
        ckv = w["dkv"] @ h[t]
        c = rms_norm(ckv[:rank], w["dkv.norm"], eps)
        kr_all.append(rotate(ckv[rank:], positions[t], rdims, base))
        k_all.append((w["uk"] @ c).reshape(H, dim))
        v_all.append((w["uv"] @ c).reshape(H, vdim))
        q_all.append(q)
        gate_all.append(sigmoid(w["g"] @ h[t]))
    out = np.zeros((T, w["o"].shape[0]))
    for t in range(T):
        heads = []
        for i in range(H):
            keys = [j for j in range(T) if 0 <= positions[t] - positions[j] < window and j <= t]
            s = np.array([(q_all[t][i, :dim] @ k_all[j][i] + q_all[t][i, dim:] @ kr_all[j]) * scale for j in keys])
            p = np.exp(s - s.max())
            p /= p.sum()
            o = sum(pj * v_all[j][i] for pj, j in zip(p, keys))
            heads.append(o * gate_all[t][i])
        out[t] = w["o"] @ np.concatenate(heads)
    return out


# ------------------------------------------------------------------------------------------------ feed-forward #
def route(h: np.ndarray, router_w: np.ndarray, correction: np.ndarray, r: dict) -> tuple[list[int], np.ndarray]:
    """Chosen experts (by descending choice score) and their normalised weights for one token."""
    E, top = r["experts"], r["top"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    s = sigmoid(router_w @ h)
    choice = s + correction
    per = E // groups["count"]
    gscore = []
    for g in range(groups["count"]):
        part = sorted(choice[g * per:(g + 1) * per], reverse=True)
        gscore.append(sum(part[:2]))
    kept = sorted(range(groups["count"]), key=lambda g: (-gscore[g], g))[:groups["keep"]]
    masked = np.full(E, -np.inf)
    for g in kept:
        masked[g * per:(g + 1) * per] = choice[g * per:(g + 1) * per]
    chosen = sorted(range(E), key=lambda e: (-masked[e], e))[:top]
    weights = np.array([s[e] for e in chosen])
    return chosen, weights / (weights.sum() + 1e-20)


def expert(h: np.ndarray, up: np.ndarray, down: np.ndarray) -> np.ndarray:
    return down @ gelu_erf(up @ h)


def moe(h: np.ndarray, spec: dict, w: dict) -> np.ndarray:
    """One token through the routed experts and the shared one."""
    chosen, weights = route(h, w["router"], w["correction"], spec["router"])
    out = np.zeros(w["e0.down"].shape[0])
    for e, g in zip(chosen, weights):
        out += g * expert(h, w[f"e{e}.up"], w[f"e{e}.down"])
    if spec.get("shared"):
        out += expert(h, w["shared.up"], w["shared.down"])
    return out


# ------------------------------------------------------------------------------------------------- whole model #
def _sub(tensors: dict, prefix: str) -> dict:
    return {k[len(prefix):]: f64(v) for k, v in tensors.items() if k.startswith(prefix)}


def source_layer(config: dict, i: int) -> int:
    while config["layers"][i].get("weights_of") is not None:
        i = config["layers"][i]["weights_of"]
    return i


def forward(config: dict, tensors: dict, tokens: list[int], trace: list | None = None) -> np.ndarray:
    """Logits ``[T, vocab]`` of one whole sequence; ``trace`` collects the residual stream after every layer."""
    eps = float(config["norm"]["eps"])
    T = len(tokens)
    pos = list(range(T))
    x = f64(tensors["embed"])[tokens] * float(config["embedding"]["scale"])
    for i, layer in enumerate(config["layers"]):
        j = source_layer(config, i)
        p = f"l{j}."
        n1, n1b = f64(tensors[p + "norm1"]), f64(tensors[p + "norm1b"])
        ls1 = f64(tensors[p + "ls1"])
        if layer["type"] != "latent_attention":
            raise ValueError(layer["type"])
        h = np.stack([layer_norm(x[t], n1, eps) for t in range(T)])
        y = latent_attention(h, pos, layer["mixer"], _sub(tensors, p + "mix."), eps)
        x = x + np.stack([layer_norm(y[t], n1b, eps) * ls1 for t in range(T)])
        if layer.get("mlp") is not None:
            n2, n2b = f64(tensors[p + "norm2"]), f64(tensors[p + "norm2b"])
            ls2 = f64(tensors[p + "ls2"])
            mw = _sub(tensors, p + "mlp.")
            y = np.stack([moe(layer_norm(x[t], n2, eps), layer["mlp"], mw) for t in range(T)])
            x = x + np.stack([layer_norm(y[t], n2b, eps) * ls2 for t in range(T)])
        if trace is not None:
            trace.append(x.copy())
    fin = f64(tensors["final.norm"])
    head = f64(tensors["head"])
    logits = np.stack([head @ layer_norm(x[t], fin, eps) for t in range(T)])
    return soft_cap(logits, float(config.get("logit_softcap") or 0.0))
