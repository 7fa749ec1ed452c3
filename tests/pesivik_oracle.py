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


def route_margin(h: np.ndarray, router_w: np.ndarray, correction: np.ndarray, r: dict) -> float:
    """How far the choice is from going another way: the smaller of the gap between the last kept and the first dropped
    group and the gap between the last chosen and the first unchosen eligible expert (inf where there is no rival)."""
    E, top = r["experts"], r["top"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    choice = sigmoid(router_w @ h) + correction
    per = E // groups["count"]
    gscore = [sum(sorted(choice[g * per:(g + 1) * per], reverse=True)[:2]) for g in range(groups["count"])]
    order = sorted(range(groups["count"]), key=lambda g: (-gscore[g], g))
    kept = order[:groups["keep"]]
    gap = gscore[order[groups["keep"] - 1]] - gscore[order[groups["keep"]]] if groups["keep"] < groups["count"] else math.inf
    eligible = sorted((choice[e] for g in kept for e in range(g * per, (g + 1) * per)), reverse=True)
    if top < len(eligible):
        gap = min(gap, eligible[top - 1] - eligible[top])
    return float(gap)


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


def forward(config: dict, tensors: dict, tokens: list[int], trace: list | None = None,
            margins: list | None = None) -> np.ndarray:
    """Logits ``[T, vocab]`` of one whole sequence; ``trace`` collects the residual stream after every layer,
    ``margins`` one array ``[T]`` of routing margins per routed layer."""
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
            if margins is not None:
                margins.append(np.array([route_margin(layer_norm(x[t], n2, eps), mw["router"], mw["correction"],
                                                      layer["mlp"]["router"]) for t in range(T)]))
            x = x + np.stack([layer_norm(y[t], n2b, eps) * ls2 for t in range(T)])
        if trace is not None:
            trace.append(x.copy())
    fin = f64(tensors["final.norm"])
    head = f64(tensors["head"])
    logits = np.stack([head @ layer_norm(x[t], fin, eps) for t in range(T)])
    return soft_cap(logits, float(config.get("logit_softcap") or 0.0))


# ------------------------------------------------------------------------------------- test models of any size #
def mixer_entry(heads=3, dim=8, rot_dim=4, vdim=10, q_rank=20, kv_rank=12, window=7, base=10000.0, scale=None) -> dict:
    return {"dim": dim, "heads": heads, "kv_rank": kv_rank, "mask": {"size": window}, "q_rank": q_rank,
            "rot": {"base": base, "dims": rot_dim}, "rot_dim": rot_dim,
            "scale": scale if scale is not None else 1.0 / math.sqrt(dim + rot_dim), "vdim": vdim}


def moe_entry(experts=8, top=3, groups=4, keep=2, ff=12, shared_ff=20) -> dict:
    out = {"expert": {"ff": ff}, "kind": "moe", "router": {"experts": experts, "groups": {"count": groups, "keep": keep},
                                                            "top": top}}
    if shared_ff:
        out["shared"] = {"ff": shared_ff}
    return out


def layer_entry(mixer: dict, mlp: dict | None, weights_of: int | None = None) -> dict:
    out = {"type": "latent_attention", "mixer": mixer, "mlp": mlp}
    if weights_of is not None:
        out["weights_of"] = weights_of
    return out


def make_config(layers: list[dict], width=48, vocab=50, eps=1e-5, embed_scale=0.7, softcap=12.0) -> dict:
    return {"architecture": "Pesivik", "embedding": {"scale": embed_scale}, "layers": layers, "logit_softcap": softcap,
            "norm": {"eps": eps}, "vocab": vocab, "width": width}


def random_model(config: dict, seed: int = 0, spread: float = 1.0):
    """Random tensors with checkpoint names, already rounded to bfloat16 values (returned as float32 torch tensors)."""
    import torch

    g = torch.Generator().manual_seed(seed)
    w = config["width"]

    def mat(rows, cols, gain=1.0):
        return torch.randn(rows, cols, generator=g) * (gain * spread / math.sqrt(cols))

    def vec(n, centre, dev):
        return centre + dev * torch.randn(n, generator=g)

    t = {"embed": torch.randn(config["vocab"], w, generator=g), "final.norm": vec(w, 1.0, 0.1),
         "head": mat(config["vocab"], w, 3.0)}
    for i, layer in enumerate(config["layers"]):
        if layer.get("weights_of") is not None:
            continue
        m, p = layer["mixer"], f"l{i}."
        H, dim, rot, vdim, qr, kr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["q_rank"], m["kv_rank"]
        t.update({p + "norm1": vec(w, 1.0, 0.1), p + "norm1b": vec(w, 1.0, 0.1), p + "ls1": vec(w, 0.5, 0.1),
                  p + "mix.dq": mat(qr, w), p + "mix.dq.norm": vec(qr, 1.0, 0.1), p + "mix.uq": mat(H * (dim + rot), qr, 2.0),
                  p + "mix.dkv": mat(kr + rot, w), p + "mix.dkv.norm": vec(kr, 1.0, 0.1),
                  p + "mix.uk": mat(H * dim, kr, 2.0), p + "mix.uv": mat(H * vdim, kr), p + "mix.g": mat(H, w, 2.0),
                  p + "mix.o": mat(w, H * vdim)})
        if layer.get("mlp") is not None:
            f, r = layer["mlp"], layer["mlp"]["router"]
            t.update({p + "norm2": vec(w, 1.0, 0.1), p + "norm2b": vec(w, 1.0, 0.1), p + "ls2": vec(w, 0.5, 0.1),
                      p + "mlp.router": mat(r["experts"], w, 2.0), p + "mlp.correction": vec(r["experts"], -0.3, 0.4)})
            for e in range(r["experts"]):
                t[f"{p}mlp.e{e}.up"], t[f"{p}mlp.e{e}.down"] = mat(f["expert"]["ff"], w), mat(w, f["expert"]["ff"])
            if f.get("shared"):
                t[p + "mlp.shared.up"], t[p + "mlp.shared.down"] = mat(f["shared"]["ff"], w), mat(w, f["shared"]["ff"])
    return {k: v.to(torch.bfloat16).float() for k, v in t.items()}
