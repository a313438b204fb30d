"""A plain, slow restatement of the reference's Llama path, for the tests only.

It rests on the reference's formulas: the reference's own model code is Java
that needs a JVM and a GGUF parser package that its tree does not hold, so it
can be neither compiled nor imported here, and nothing under tests/golden/
comes from running it.

Whole sequences, no cache, one function for each part; it imports nothing from
the library under test. Paths cite the reference by its project-relative name
(all under src/main/java/it/denzosoft/llmplayer/ unless they start with
src/main/resources/).
"""
from __future__ import annotations

import json
import math
import os
import struct

import torch


# --------------------------------------------------------------------------- files
def read_safetensors(path):
    """Minimal reader of the container, independent of the library's own."""
    with open(path, "rb") as fh:
        (hlen,) = struct.unpack("<Q", fh.read(8))
        header = json.loads(fh.read(hlen))
        data = fh.read()
    kinds = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16, "I32": torch.int32}
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        t = torch.frombuffer(bytearray(data[b:e]), dtype=torch.uint8).view(kinds[info["dtype"]])
        out[name] = t.reshape(info["shape"]).clone()
    return out


def read_model(model_dir):
    with open(os.path.join(model_dir, "config.json")) as fh:
        cfg = json.load(fh)
    return cfg, read_safetensors(os.path.join(model_dir, "model.safetensors"))


# --------------------------------------------------------------------------- parts
def rms_norm(x, weight, eps):
    """out_i = x_i * (1 / sqrt(mean(x^2) + eps)) * w_i — tensor/ScalarOps.java:26-35,
    src/main/resources/kernels/cuda/rmsnorm.cu:19-45. The gain is used as stored."""
    ss = (x * x).sum(dim=-1, keepdim=True)
    r = 1.0 / torch.sqrt(ss / x.shape[-1] + eps)
    return x * r * weight


def rope_inverse_frequencies(rotary_dim, theta, scaling=None):
    """f_i = 1 / theta^(2i/rotary_dim), computed in double and rounded to float32 —
    inference/RoPE.java:83. The reference divides f_i by a per-pair factor read
    from the file (inference/RoPE.java:85-87, model/ModelLoader.java:675-693);
    for "llama3" scaling that factor comes from the wavelength rule below, which
    the file's converter applies: wavelengths shorter than original/high stay,
    longer than original/low are stretched by ``factor``, between them blended."""
    out = []
    for i in range(rotary_dim // 2):
        f = 1.0 / math.pow(theta, 2.0 * i / rotary_dim)
        if scaling is not None:
            factor = float(scaling["factor"])
            low = float(scaling["low_freq_factor"])
            high = float(scaling["high_freq_factor"])
            orig = float(scaling["original_max_position_embeddings"])
            wavelen = 2.0 * math.pi / f
            if wavelen < orig / high:
                pass
            elif wavelen > orig / low:
                f = f / factor
            else:
                s = (orig / wavelen - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return torch.tensor(out, dtype=torch.float64).to(torch.float32)


def rope_rotate(x, positions, inv_freq, pairing="split_half"):
    """x: [T, heads, head_dim]. angle = position * f_i as a float32 product, cos and sin
    evaluated in double on that angle (inference/RoPE.java:101-104); pair (a, b) becomes
    (a cos - b sin, a sin + b cos) (inference/RoPE.java:158-168 for split halves,
    :148-156 for neighbours)."""
    rd = inv_freq.numel() * 2
    angle = positions.to(torch.float32)[:, None] * inv_freq[None, :]          # float32 product
    cos = torch.cos(angle.to(torch.float64)).to(x.dtype)[:, None, :]
    sin = torch.sin(angle.to(torch.float64)).to(x.dtype)[:, None, :]
    out = x.clone()
    if pairing == "split_half":
        a, b = x[..., : rd // 2], x[..., rd // 2: rd]
        out[..., : rd // 2] = a * cos - b * sin
        out[..., rd // 2: rd] = a * sin + b * cos
    else:
        a, b = x[..., 0:rd:2], x[..., 1:rd:2]
        out[..., 0:rd:2] = a * cos - b * sin
        out[..., 1:rd:2] = a * sin + b * cos
    return out


def attention(q, k, v, scale, window=None, q_positions=None):
    """q: [Tq, H, hd]; k, v: [Tk, G, hd] for positions 0..Tk-1; query head h uses KV
    head h // (H/G). Scores (q.k)*scale over keys t <= p, softmax with the maximum
    subtracted, weighted sum of values in increasing t — inference/Attention.java:138-140,
    :210-230; src/main/resources/kernels/cuda/attention.cu:26-107. ``window`` keeps
    keys with t > p - window."""
    Tq, H, hd = q.shape
    Tk, G, _ = k.shape
    if q_positions is None:
        q_positions = torch.arange(Tk - Tq, Tk)
    out = torch.zeros_like(q)
    rep = H // G
    t = torch.arange(Tk)
    for h in range(H):
        g = h // rep
        s = (q[:, h, :] @ k[:, g, :].T) * scale                               # [Tq, Tk]
        allowed = t[None, :] <= q_positions[:, None]
        if window is not None:
            allowed &= t[None, :] > (q_positions[:, None] - window)
        s = s.masked_fill(~allowed, float("-inf"))
        m = s.max(dim=-1, keepdim=True).values
        e = torch.exp(s - m)
        a = e * (1.0 / e.sum(dim=-1, keepdim=True))
        out[:, h, :] = a @ v[:, g, :]
    return out


def swiglu(x, w_gate, w_up, w_down):
    """down(silu(gate x) * (up x)), silu(g) = g / (1 + exp(-g)) —
    inference/SwiGLUFFN.java:36-67, tensor/ScalarOps.java:69-73."""
    g = x @ w_gate.T
    u = x @ w_up.T
    return ((g / (1.0 + torch.exp(-g))) * u) @ w_down.T


def attention_block(x, w, prefix, cfg, inv_freq, positions, window=None):
    """QKV projections without bias, rotation of q and k, attention, output projection —
    inference/Attention.java:86-135, :234-239."""
    H = cfg["num_attention_heads"]
    G = cfg.get("num_key_value_heads") or H
    hd = cfg.get("head_dim") or cfg["hidden_size"] // H
    T = x.shape[0]
    q = (x @ w[prefix + "self_attn.q_proj.weight"].T).reshape(T, H, hd)
    k = (x @ w[prefix + "self_attn.k_proj.weight"].T).reshape(T, G, hd)
    v = (x @ w[prefix + "self_attn.v_proj.weight"].T).reshape(T, G, hd)
    q = rope_rotate(q, positions, inv_freq)
    k = rope_rotate(k, positions, inv_freq)
    o = attention(q, k, v, 1.0 / math.sqrt(hd), window=window, q_positions=positions)
    return o.reshape(T, H * hd) @ w[prefix + "self_attn.o_proj.weight"].T


def forward(cfg, tensors, tokens, dtype=torch.float64, layers=None, rows=None):
    """Logits [T, vocab] of one whole sequence (or of its positions ``rows`` only, which spares
    a large vocabulary's head for the others): embedding row without scaling
    (inference/InferenceEngine.java:199-208), for each layer x += attention(norm(x)),
    x += ffn(norm(x)) (inference/TransformerBlock.java:73-149), final norm and head,
    which is the embedding table when tied (inference/InferenceEngine.java:225-262,
    model/ModelLoader.java:207-214)."""
    w = {k: v.to(dtype) for k, v in tensors.items()}
    H = cfg["num_attention_heads"]
    hd = cfg.get("head_dim") or cfg["hidden_size"] // H
    eps = cfg["rms_norm_eps"]
    inv_freq = rope_inverse_frequencies(hd, cfg["rope_theta"], cfg.get("rope_scaling"))
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(tokens.numel())
    x = w["model.embed_tokens.weight"][tokens]
    n_layers = cfg["num_hidden_layers"] if layers is None else layers
    for i in range(n_layers):
        p = f"model.layers.{i}."
        x = x + attention_block(rms_norm(x, w[p + "input_layernorm.weight"], eps), w, p, cfg, inv_freq, positions)
        h = rms_norm(x, w[p + "post_attention_layernorm.weight"], eps)
        x = x + swiglu(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    if rows is not None:
        x = x[torch.as_tensor(rows, dtype=torch.long)]
    x = rms_norm(x, w["model.norm.weight"], eps)
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else w["lm_head.weight"]
    return x @ head.T


def greedy_generate(cfg, tensors, prompt, steps, stop_ids=(), dtype=torch.float64):
    """Sample from the last logits, stop at an end token without emitting it, else append
    and run again — api/LLMEngine.java:743-769 (here each run is a whole-sequence pass)."""
    seq = list(prompt)
    out = []
    for _ in range(steps):
        logits = forward(cfg, tensors, seq, dtype=dtype)[-1]
        nxt = argmax_first(logits)
        if nxt in stop_ids:
            break
        out.append(nxt)
        seq.append(nxt)
    return out


# --------------------------------------------------------------------------- sampling
def argmax_first(values):
    """First maximum wins (strict >) — sampler/CompositeSampler.java:259-269."""
    best, best_val = 0, float(values[0])
    vals = values.tolist()
    for i in range(1, len(vals)):
        if vals[i] > best_val:
            best, best_val = i, vals[i]
    return best


class JavaRandom:
    """java.util.Random: 48-bit linear congruential generator; nextFloat() is the top
    24 bits over 2^24. The reference seeds one per request (sampler/CompositeSampler.java:24)."""

    def __init__(self, seed):
        self.state = (int(seed) ^ 0x5DEECE66D) & ((1 << 48) - 1)

    def next_bits(self, bits):
        self.state = (self.state * 0x5DEECE66D + 0xB) & ((1 << 48) - 1)
        return self.state >> (48 - bits)

    def next_float(self):
        return self.next_bits(24) / float(1 << 24)


def f32(x):
    return struct.unpack("<f", struct.pack("<f", x))[0]


class PlainSampler:
    """sampler/CompositeSampler.java:33-120 in float32 arithmetic, step by step:
    DRY penalty, repetition penalty, greedy if temperature is 0, else scale by 1/T,
    top-k by threshold (ties at the threshold survive), softmax, min-p, top-p,
    then mirostat v2 or an inverse-CDF walk in index order."""

    def __init__(self, temperature=0.7, top_k=40, top_p=0.9, repetition_penalty=1.1, seed=0, min_p=0.0,
                 mirostat=0, mirostat_tau=5.0, mirostat_eta=0.1, dry_multiplier=0.0, dry_base=1.75,
                 dry_allowed_length=2, dry_range=1024):
        self.c = dict(locals())
        self.rng = JavaRandom(seed)
        self.recent = []
        self.max_recent = max(64, dry_range)
        self.mu = f32(2.0 * mirostat_tau)

    def _remember(self, tok):
        self.recent.append(tok)
        if len(self.recent) > self.max_recent:
            self.recent.pop(0)

    def sample(self, logits):
        c = self.c
        p = logits.detach().to(torch.float32).cpu().clone()
        V = p.numel()
        if c["dry_multiplier"] > 0:
            self._dry(p)
        if c["repetition_penalty"] != 1.0:
            r = torch.tensor(c["repetition_penalty"], dtype=torch.float32)
            for tok in self.recent:                      # once per occurrence, as the reference does
                if 0 <= tok < V:
                    p[tok] = p[tok] / r if p[tok] > 0 else p[tok] * r
        if c["temperature"] == 0.0:
            tok = argmax_first(p)
            self._remember(tok)
            return tok
        p = p * torch.tensor(1.0 / f32(c["temperature"]), dtype=torch.float32)
        k = c["top_k"]
        if k <= 0 or k >= V:
            k = V
        if k < V:
            thr = torch.sort(p, descending=True).values[k - 1]
            p = torch.where(p < thr, torch.tensor(float("-inf")), p)
        m = p.max()
        e = torch.where(torch.isinf(p) & (p < 0), torch.zeros_like(p), torch.exp(p - m))
        s = e.sum()
        if s > 0:
            e = e * (1.0 / s)
        if c["min_p"] > 0:
            mx = e.max()
            if mx > 0:
                e = torch.where(e < f32(c["min_p"]) * mx, torch.zeros_like(e), e)
                s = e.sum()
                if s > 0:
                    e = e * (1.0 / s)
        if c["top_p"] < 1.0:
            e = self._top_p(e, f32(c["top_p"]))
        tok = self._mirostat(e) if c["mirostat"] == 2 else self._multinomial(e)
        self._remember(tok)
        return tok

    @staticmethod
    def _order(e):
        """Indices of the non-zero entries, descending by probability, equal ones in index order."""
        idx = torch.nonzero(e > 0).flatten()
        vals = e[idx]
        order = torch.sort(vals, descending=True, stable=True).indices
        return idx[order]

    def _top_p(self, e, top_p):
        idx = self._order(e)
        if idx.numel() <= 1:
            return e
        cum = torch.cumsum(e[idx], dim=0)
        over = torch.nonzero(cum > top_p).flatten()
        cutoff = int(over[0]) + 1 if over.numel() else idx.numel()
        keep = torch.zeros_like(e)
        keep[idx[:cutoff]] = e[idx[:cutoff]]
        s = keep.sum()
        return keep * (1.0 / s) if s > 0 else keep

    def _multinomial(self, e):
        r = self.rng.next_float()
        cum = torch.cumsum(e, dim=0)
        hit = torch.nonzero(cum > r).flatten()
        return int(hit[0]) if hit.numel() else e.numel() - 1

    def _mirostat(self, e):
        idx = self._order(e)
        if idx.numel() == 0:
            return self._multinomial(e)
        thr = f32(math.pow(2.0, -self.mu))
        keep = int((e[idx] >= thr).sum())
        keep = max(keep, 1)
        idx = idx[:keep]
        s = float(e[idx].sum())
        if s <= 0:
            return int(idx[0])
        r = f32(self.rng.next_float() * s)
        cum = torch.cumsum(e[idx], dim=0)
        hit = torch.nonzero(cum > r).flatten()
        tok = int(idx[int(hit[0])]) if hit.numel() else int(idx[0])
        observed = float(e[tok]) / s
        surprise = f32(-(math.log(observed) / math.log(2.0)))
        self.mu = f32(self.mu - f32(self.c["mirostat_eta"]) * f32(surprise - f32(self.c["mirostat_tau"])))
        return tok

    def _dry(self, p):
        """sampler/CompositeSampler.java:150-192."""
        c, rec = self.c, self.recent
        n = len(rec)
        if n < 2:
            return
        rng = min(n, c["dry_range"])
        start = n - rng
        last = rec[n - 1]
        for pos in range(start, n - 1):
            if rec[pos] != last:
                continue
            match, pi, ni = 1, pos - 1, n - 2
            while pi >= start and ni > pos and rec[pi] == rec[ni]:
                match, pi, ni = match + 1, pi - 1, ni - 1
            nxt = rec[pos + 1]
            if 0 <= nxt < p.numel() and match >= c["dry_allowed_length"]:
                p[nxt] -= f32(f32(c["dry_multiplier"]) * f32(math.pow(c["dry_base"], match - c["dry_allowed_length"])))
