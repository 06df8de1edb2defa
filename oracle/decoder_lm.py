"""Plain, slow restatement of the text-only decoder LM (the Likosun design) in float64: one function per mechanism, written
from the equations and sharing no code with ``moshi_b200``.  Keys and values are materialised per head here (the product path
never does that: it scores against the cached latent), so agreement between the two checks the algebra as well.

Notation: h = normed layer input [T, W]; c = latent [T, r]; per head q, k [dim], v [vdim]; s = sink logit of the head.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def layer_norm(x, w, b, eps):
    """(x - mean) / sqrt(mean((x - mean)^2) + eps) * w + b over the last axis."""
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def sink_softmax(scores, sink):
    """Softmax over the last axis whose denominator holds one more term exp(sink) that belongs to no key.  -inf scores drop out."""
    m = torch.maximum(scores.max(-1, keepdim=True).values, sink)
    e = torch.exp(scores - m)
    return e / (e.sum(-1, keepdim=True) + torch.exp(sink - m))


def latent(h, w_dkv, w_norm, eps):
    """c = rms_norm(W_dkv h)."""
    return rms_norm(h @ w_dkv.T, w_norm, eps)


def latent_attention(h, c_all, pos0, P, heads, dim, vdim, scale):
    """Causal attention of the T rows of ``h`` (positions pos0 .. pos0 + T - 1) over the latents ``c_all`` [pos0 + T, r].
    P: dict with q, uk, uv, sink, o.  No positional signal of any kind."""
    T = h.shape[0]
    n = c_all.shape[0]
    q = (h @ P["q"].T).view(T, heads, dim)
    k = (c_all @ P["uk"].T).view(n, heads, dim)
    v = (c_all @ P["uv"].T).view(n, heads, vdim)
    out = torch.zeros(T, heads, vdim, dtype=h.dtype)
    for t in range(T):
        last = pos0 + t
        for hd in range(heads):
            s = (k[:last + 1, hd] @ q[t, hd]) * scale
            p = sink_softmax(s[None, :], P["sink"][hd].reshape(1, 1))[0]
            out[t, hd] = p @ v[:last + 1, hd]
    return out.reshape(T, heads * vdim) @ P["o"].T


def relu2_mlp(h, up, down):
    """W_down relu(W_up h)^2."""
    return (torch.relu(h @ up.T) ** 2) @ down.T


def gate(h, y, G, g):
    """y * sigmoid(G h + g), element by element."""
    return y * torch.sigmoid(h @ G.T + g)


def depth_average(results, a):
    """sum_j a[j] * results[j]."""
    return sum(a[j] * results[j] for j in range(len(results)))


class DecoderOracle:
    """Whole model; ``forward`` takes new tokens of ONE request on top of what earlier calls left in ``state``."""

    def __init__(self, cfg, tensors):
        self.cfg = cfg
        self.W = {k: v.to(F64) for k, v in dict(tensors).items()}

    def new_state(self):
        return {"c": [torch.zeros(0, L.kv_rank, dtype=F64) for L in self.cfg.layers]}

    def forward(self, tokens, state=None, return_layers=False):
        cfg, W = self.cfg, self.W
        state = self.new_state() if state is None else state
        pos0 = state["c"][0].shape[0]
        x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)] * cfg.embedding_scale
        results, handed = [x], []
        for i, L in enumerate(cfg.layers):
            p = f"l{i}."
            h = layer_norm(x, W[p + "norm1"], W[p + "norm1.b"], cfg.norm_eps)
            c = latent(h, W[p + "mix.dkv"], W[p + "mix.dkv.norm"], cfg.norm_eps)
            state["c"][i] = torch.cat([state["c"][i], c])
            P = {k: W[p + "mix." + k] for k in ("q", "uk", "uv", "sink", "o")}
            y = gate(h, latent_attention(h, state["c"][i], pos0, P, L.heads, L.dim, L.vdim, L.scale), W[p + "rg1"], W[p + "rg1.b"])
            if L.mlp_kind is not None:
                y = y + gate(h, relu2_mlp(h, W[p + "mlp.up"], W[p + "mlp.down"]), W[p + "rg2"], W[p + "rg2.b"])
            results.append(x + cfg.residual_mult * y)
            x = depth_average(results, W[p + "dwa"])
            handed.append(x)
        logits = layer_norm(x, W["final.norm"], W["final.norm.b"], cfg.norm_eps) @ W["head"].T
        return (logits, torch.stack(handed)) if return_layers else logits

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


def logit_error(got, want):
    """Per row: rms over the vocabulary of the difference with its mean taken off, relative to the rms of the wanted logits."""
    d = got.to(F64) - want.to(F64)
    d = d - d.mean(-1, keepdim=True)
    return torch.sqrt((d * d).mean(-1)) / torch.sqrt((want.to(F64) ** 2).mean())
