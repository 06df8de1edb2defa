"""Plain, slow restatement of the Govuvik decoder LM in float64: one function per mechanism, written from the equations and
sharing no code with ``moshi_b200``.  Everything runs token by token on explicit per-request state (lists of past keys and
values, the last inputs of every causal convolution, the matrices of the two recurrences), with no tiling, chunking or fused
step of any kind, so agreement with the product path checks its kernels, its cache and its state handling alike.

Notation: x residual stream [W]; h what a sublayer reads; per head q, k [dim], v [vdim]; S matrix memory [dim, vdim].
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis (w may be None: no weight)."""
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def causal_conv_step(history, u, w):
    """One step of a per-channel causal convolution.  ``history``: list of the earlier inputs (newest last, may be shorter than
    taps - 1 at the start of a sequence: missing inputs are zero); w [C, taps]; the newest input meets the last tap."""
    taps = w.shape[1]
    y = w[:, taps - 1] * u
    for back in range(1, taps):
        if back <= len(history):
            y = y + w[:, taps - 1 - back] * history[-back]
    return y


def rope_frequencies(dims, base, scaling):
    """f_i = base^(-2i/dims), i < dims/2, rescaled by wavelength: short waves keep f, long waves get f / factor, and the band
    between original/high and original/low is blended linearly in original/wavelength."""
    out = []
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if scaling is not None:
            factor, low, high, orig = scaling["factor"], scaling["low"], scaling["high"], scaling["original"]
            wave = 2.0 * math.pi / f
            if wave < orig / high:
                pass
            elif wave > orig / low:
                f = f / factor
            else:
                s = (orig / wave - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return torch.tensor(out, dtype=F64)


def rope_rotate(u, pos, freqs):
    """u [heads, dim]: the first 2 * len(freqs) dimensions of every head are rotated, dimension i with i + len(freqs)."""
    half = freqs.shape[0]
    ang = pos * freqs
    c, s = torch.cos(ang), torch.sin(ang)
    a, b = u[:, :half], u[:, half:2 * half]
    out = u.clone()
    out[:, :half] = a * c - b * s
    out[:, half:2 * half] = b * c + a * s
    return out


def mixed_window_attention(q, keys, values, pos, window, scale, temp, talk, sink):
    """One query token.  q [H, dim]; keys / values: lists of [G, dim] / [G, vdim] for positions 0 .. pos; the token sees the last
    ``window`` of them (itself included).  Raw scores are scaled, multiplied by the head's temperature, then mixed over heads by
    ``talk`` [H, H]; the softmax denominator has one more term exp(sink[h])."""
    H = q.shape[0]
    G = keys[0].shape[0]
    lo = max(0, pos - window + 1)
    k, v = torch.stack(keys[lo:pos + 1]), torch.stack(values[lo:pos + 1])
    rep = H // G
    raw = torch.stack([(k[:, h // rep] @ q[h]) * scale * temp[h] for h in range(H)])      # [H, n]
    s = talk @ raw
    m = torch.maximum(s.max(-1).values, sink)
    e = torch.exp(s - m[:, None])
    p = e / (e.sum(-1) + torch.exp(sink - m))[:, None]
    return torch.stack([p[h] @ v[:, h // rep] for h in range(H)])                         # [H, vdim]


def gla_step(S, q, k, v, alpha):
    """S [heads, dim, vdim] <- diag(alpha) S + k v^T per head; returns (S, o = S^T q)."""
    S = alpha[:, :, None] * S + k[:, :, None] * v[:, None, :]
    return S, torch.einsum("hdv,hd->hv", S, q)


def mlstm_step(S, n, m, q, k, v, i_log, f_log):
    """Stabilised matrix memory, per head: m' = max(f + m, i); S' = e^(f + m - m') S + e^(i - m') k v^T, n' likewise with k;
    o = S'^T q / (max(|n' . q|, e^(-m')) + 1e-6)."""
    m2 = torch.maximum(f_log + m, i_log)
    a, b = torch.exp(f_log + m - m2), torch.exp(i_log - m2)
    S = a[:, None, None] * S + b[:, None, None] * k[:, :, None] * v[:, None, :]
    n = a[:, None] * n + b[:, None] * k
    num = torch.einsum("hdv,hd->hv", S, q)
    den = torch.maximum((n * q).sum(-1).abs(), torch.exp(-m2)) + 1e-6
    return S, n, m2, num / den[:, None]


def capped(z, cap):
    return cap * torch.tanh(z / cap)


def moe_relu2(h, router, ups, downs, top):
    """The ``top`` experts with the largest router logits, weighted by the softmax over those logits alone; expert = W_down relu(W_up h)^2."""
    z = router @ h
    val, idx = torch.topk(z, top)
    w = torch.softmax(val, -1)
    return sum(w[j] * (downs[int(e)] @ (torch.relu(ups[int(e)] @ h) ** 2)) for j, e in enumerate(idx))


def softcap(z, cap):
    return cap * torch.tanh(z / cap)


class GovuvikOracle:
    """Whole model.  ``cfg`` is the raw ``config.json`` dictionary; ``forward`` takes new tokens of ONE request on top of ``state``."""

    def __init__(self, cfg: dict, tensors):
        self.cfg = cfg
        self.W = {k: v.to(F64) for k, v in dict(tensors).items()}
        self.eps = float(cfg["norm"]["eps"])
        self.freqs = {}
        for i, L in enumerate(cfg["layers"]):
            if L["type"] == "parallel":
                rot = L["mixer"]["left"]["rot"]
                self.freqs[i] = rope_frequencies(int(rot["dims"]), float(rot["base"]), rot.get("scaling"))

    def new_state(self):
        st = {"pos": 0, "layers": []}
        for L in self.cfg["layers"]:
            m = L["mixer"]
            if L["type"] == "parallel":
                l, r = m["left"], m["right"]
                st["layers"].append({"canon": [], "q": [], "k": [], "v": [], "keys": [], "values": [],
                                     "S": torch.zeros(r["heads"], r["dim"], r["vdim"], dtype=F64)})
            else:
                st["layers"].append({"canon": [], "S": torch.zeros(m["heads"], m["dim"], m["vdim"], dtype=F64),
                                     "n": torch.zeros(m["heads"], m["dim"], dtype=F64), "m": torch.zeros(m["heads"], dtype=F64)})
        return st

    @staticmethod
    def _push(history, u, keep):
        history.append(u)
        while len(history) > keep:
            del history[0]

    def _parallel(self, i, m, h, pos, st):
        W, p, eps = self.W, f"l{i}.mix.", self.eps
        l, r = m["left"], m["right"]
        H, G, dim, vdim = l["heads"], l["kv_heads"], l["dim"], l["vdim"]
        proj = {}
        for name in ("q", "k", "v"):
            u = W[p + f"left.{name}"] @ h
            if int(l.get("conv", 0)) >= 1:
                proj[name] = causal_conv_step(st[name], u, W[p + f"left.{name}.conv"])
                self._push(st[name], u, int(l["conv"]) - 1)
            else:
                proj[name] = u
        q = rms_norm(proj["q"], W[p + "left.q.norm"], eps).view(H, dim)
        k = rms_norm(proj["k"], W[p + "left.k.norm"], eps).view(G, dim)
        q, k = rope_rotate(q, pos, self.freqs[i]), rope_rotate(k, pos, self.freqs[i])
        st["keys"].append(k)
        st["values"].append(proj["v"].view(G, vdim))
        o = mixed_window_attention(q, st["keys"], st["values"], pos, int(l["mask"]["size"]), float(l["scale"]),
                                   W[p + "left.temp"], W[p + "left.talk"], W[p + "left.sink"])
        left = W[p + "left.o"] @ o.reshape(-1)
        # gated linear attention
        Hr, dr, vr = r["heads"], r["dim"], r["vdim"]
        q2 = (W[p + "right.q"] @ h).view(Hr, dr) * dr ** -0.5
        k2 = (W[p + "right.k"] @ h).view(Hr, dr)
        v2 = (W[p + "right.v"] @ h).view(Hr, vr)
        z = W[p + "right.a2"] @ (W[p + "right.a1"] @ h) + W[p + "right.a2.b"]
        alpha = torch.sigmoid(z).pow(1.0 / float(r["tau"])).view(Hr, dr)
        st["S"], o2 = gla_step(st["S"], q2, k2, v2, alpha)
        o2 = rms_norm(o2, W[p + "right.norm"], eps).reshape(-1) * torch.nn.functional.silu(W[p + "right.g"] @ h)
        right = W[p + "right.o"] @ o2
        return 0.5 * (rms_norm(left, W[p + "left.out"], eps) + rms_norm(right, W[p + "right.out"], eps))

    def _mlstm(self, i, m, h, st):
        W, p, eps = self.W, f"l{i}.mix.", self.eps
        H, dim, vdim, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
        q = (W[p + "q"] @ h).view(H, dim) * dim ** -0.5
        k = (W[p + "k"] @ h).view(H, dim)
        v = (W[p + "v"] @ h).view(H, vdim)
        i_log = capped(W[p + "i"] @ h + W[p + "i.b"], cap)
        f_log = torch.nn.functional.logsigmoid(capped(W[p + "f"] @ h + W[p + "f.b"], cap))
        st["S"], st["n"], st["m"], o = mlstm_step(st["S"], st["n"], st["m"], q, k, v, i_log, f_log)
        o = rms_norm(o, None, eps).reshape(-1) * W[p + "norm"] * torch.sigmoid(W[p + "g"] @ h)
        return W[p + "o"] @ o

    def _token(self, tok, state, layers_out):
        cfg, W, eps = self.cfg, self.W, self.eps
        pos = state["pos"]
        x = rms_norm(W["embed"][tok], W["embed.norm"], eps)
        for i, L in enumerate(cfg["layers"]):
            p, st = f"l{i}.", state["layers"][i]
            h = rms_norm(x, W[p + "norm1"], eps)
            hc = h + causal_conv_step(st["canon"], h, W[p + "canon1"])
            self._push(st["canon"], h, int(cfg["canon"]["taps"]) - 1)
            y = self._parallel(i, L["mixer"], hc, pos, st) if L["type"] == "parallel" else self._mlstm(i, L["mixer"], hc, st)
            x = x + rms_norm(y, W[p + "norm1b"], eps)
            if L.get("mlp") is not None:
                E = int(L["mlp"]["router"]["experts"])
                h2 = rms_norm(x, W[p + "norm2"], eps)
                y = moe_relu2(h2, W[p + "mlp.router"], [W[p + f"mlp.e{e}.up"] for e in range(E)],
                              [W[p + f"mlp.e{e}.down"] for e in range(E)], int(L["mlp"]["router"]["top"]))
                x = x + rms_norm(y, W[p + "norm2b"], eps)
            layers_out.append(x)
        state["pos"] = pos + 1
        return softcap(W["head"] @ rms_norm(x, W["final.norm"], eps), float(cfg["logit_softcap"]))

    def forward(self, tokens, state=None, return_layers=False):
        state = self.new_state() if state is None else state
        logits, layers = [], []
        for t in tokens:
            per = []
            logits.append(self._token(int(t), state, per))
            layers.append(torch.stack(per))
        logits = torch.stack(logits)
        return (logits, torch.stack(layers, 1)) if return_layers else logits          # layers: [layer, token, W]

    def greedy(self, prompt, n_new):
        """(tokens, top-2 logit gaps) of greedy decoding."""
        st = self.new_state()
        lg = self.forward(prompt, st)[-1]
        out, gaps = [], []
        for _ in range(n_new):
            top = torch.topk(lg, 2).values
            out.append(int(lg.argmax()))
            gaps.append(float(top[0] - top[1]))
            lg = self.forward([out[-1]], st)[-1]
        return out, gaps
