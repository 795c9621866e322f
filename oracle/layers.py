"""Torch (CPU, fp32 by default) restatement of the reference layer forward.

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).  Each function cites the reference lines
it restates.  Weights are held in "logical" form (separate q/k/v matrices of the whole
model) so the same weights can be evaluated at any simulated tensor-parallel degree; the
helpers at the bottom convert to the reference's own state_dict naming.

Logical parameter names of one block:
    norm1.weight norm1.bias  q.weight q.bias k.weight k.bias v.weight v.bias
    dense.weight dense.bias  norm2.weight norm2.bias
    fc1.weight fc1.bias fc2.weight fc2.bias
"""
import math

import torch
import torch.nn.functional as F


def gelu_tanh(x):
    """energonai/model/model_factory.py:32-35 (gelu_impl)."""
    return 0.5 * x * (1.0 + torch.tanh(0.7978845608028654 * x * (1.0 + 0.044715 * x * x)))


ACTIVATIONS = {"relu": F.relu, "gelu_tanh": gelu_tanh, "gelu": F.gelu}


def _shard_rows(w, r, t):
    n = w.shape[0] // t
    return w[r * n:(r + 1) * n]


def _shard_cols(w, r, t):
    n = w.shape[1] // t
    return w[:, r * n:(r + 1) * n]


class OracleBlock:
    """One Block1D (energonai/model/endecoder.py:48-70) with its attention
    (attention.py:56-136) and MLP (mlp.py:30-51), evaluated for `tp` simulated ranks:
    column-parallel layers use a row shard of the weight, row-parallel layers a column shard,
    partial results are summed over ranks and the row-parallel bias is added once."""

    def __init__(self, params, num_heads, activation="relu", eps=1e-5, apply_post_layernorm=False,
                 is_decoder=True, tp=1):
        self.p = params
        self.h = params["q.weight"].shape[1]
        self.H = num_heads
        self.d = self.h // num_heads
        self.act = ACTIVATIONS[activation] if isinstance(activation, str) else activation
        self.eps = eps
        self.post_ln = apply_post_layernorm
        self.is_decoder = is_decoder
        self.tp = tp
        self.cache = [dict() for _ in range(tp)]

    # -- attention.py:56-136 for simulated rank r -------------------------------------
    def _attn_rank(self, r, x, attention_mask, first_cache):
        p, t, c = self.p, self.tp, self.cache[r]
        B = x.shape[0]
        src = x if first_cache else x[:, -1:, :]            # attention.py:51-54, 90-92
        proj = {}
        for name in ("q", "k", "v"):
            w, b = _shard_rows(p[f"{name}.weight"], r, t), _shard_rows(p[f"{name}.bias"], r, t)
            y = F.linear(src, w, b)
            c[name] = y if first_cache else torch.cat((c[name], y), 1)   # attention.py:86-98
            proj[name] = c[name]
        Hl = self.H // t
        S = proj["q"].shape[1]
        q, k, v = (proj[n].view(B, S, Hl, self.d).permute(0, 2, 1, 3) for n in ("q", "k", "v"))
        q = q * self.d ** -0.5                                # attention.py:105
        s = q @ k.transpose(-1, -2)                           # attention.py:106
        if self.is_decoder:                                   # attention.py:110-111 (replace)
            tril = torch.tril(torch.ones(S, S, dtype=torch.bool))
            s = torch.where(tril, s, torch.tensor(-1e4, dtype=s.dtype))
        if attention_mask is not None:                        # attention.py:113-114 (add)
            s = s + attention_mask
        probs = torch.softmax(s, -1, dtype=torch.float).to(s.dtype)      # attention.py:116
        ctx = (probs @ v).transpose(1, 2).reshape(B, S, Hl * self.d)     # attention.py:118-124
        w_o = _shard_cols(p["dense.weight"], r, t)
        src_o = ctx if first_cache else ctx[:, -1:, :]        # attention.py:126-135
        return F.linear(src_o, w_o)

    def attention(self, x, attention_mask, first_cache):
        part = sum(self._attn_rank(r, x, attention_mask, first_cache) for r in range(self.tp))
        y = part + self.p["dense.bias"]                       # row-parallel: bias after the sum
        c = self.cache[0]
        c["dense"] = y if first_cache else torch.cat((c["dense"], y), 1)
        return c["dense"]

    # -- mlp.py:30-51 ---------------------------------------------------------------------
    def mlp(self, x, first_cache):
        p, t = self.p, self.tp
        src = x if first_cache else x[:, -1:, :]
        part = 0
        for r in range(t):
            a = F.linear(src, _shard_rows(p["fc1.weight"], r, t), _shard_rows(p["fc1.bias"], r, t))
            part = part + F.linear(self.act(a), _shard_cols(p["fc2.weight"], r, t))
        y = part + p["fc2.bias"]
        c = self.cache[0]
        c["fc2"] = y if first_cache else torch.cat((c["fc2"], y), 1)
        return c["fc2"]

    # -- endecoder.py:48-70 ---------------------------------------------------------------
    def forward(self, x, attention_mask=None, first_cache=False):
        p = self.p
        n1 = F.layer_norm(x, (self.h,), p["norm1.weight"], p["norm1.bias"], self.eps)
        res = n1 if self.post_ln else x
        x = res + self.attention(n1, attention_mask, first_cache)
        n2 = F.layer_norm(x, (self.h,), p["norm2.weight"], p["norm2.bias"], self.eps)
        res = n2 if self.post_ln else x
        return res + self.mlp(n2, first_cache)

    __call__ = forward


class OracleModel:
    """PipelineModel.forward (energonai/model/model_factory.py:103-159) for a single pipeline
    stage: word + learned position embedding over the padded sequence (embedding.py:41-57,
    positions = arange, no offset), `depth` blocks, final LayerNorm, LM head on a separate
    weight (model_factory.py:99-101), greedy next token (top_k=1 through the reference's
    warper + multinomial is argmax up to exact ties)."""

    def __init__(self, params, depth, num_heads, activation="relu", eps=1e-5, tp=1):
        self.p = params
        self.depth, self.H, self.act, self.eps, self.tp = depth, num_heads, activation, eps, tp
        self.h = params["embed.word.weight"].shape[1]

    def _block_params(self, i):
        pre = f"blocks.{i}."
        return {k[len(pre):]: v for k, v in self.p.items() if k.startswith(pre)}

    def generate(self, input_ids, attention_mask, max_tokens, record=None):
        """Returns input_ids extended to `max_tokens` columns.  `record`, if a dict, receives
        per-step last-position logits ("logits") and the last-position hidden state of the
        final block ("hidden")."""
        p = self.p
        blocks = [OracleBlock(self._block_params(i), self.H, self.act, self.eps, tp=self.tp)
                  for i in range(self.depth)]
        B, cur = input_ids.shape
        dt = p["embed.word.weight"].dtype
        first = True
        attention_mask = attention_mask.to(dt)
        for _ in range(cur, max_tokens):
            S = input_ids.shape[1]
            x = p["embed.word.weight"][input_ids] + p["embed.pos.weight"][torch.arange(S)][None]
            m = (1.0 - attention_mask.view(B, 1, 1, S)) * -10000.0       # model_factory.py:117-121
            for blk in blocks:
                x = blk(x, m, first)
            x = F.layer_norm(x, (self.h,), p["norm.weight"], p["norm.bias"], self.eps)
            logits = F.linear(x[:, -1, :], p["head.weight"])             # generate(): logits[:, -1]
            tok = logits.argmax(-1)
            if record is not None:
                record.setdefault("logits", []).append(logits.clone())
                record.setdefault("hidden", []).append(x[:, -1, :].clone())
            input_ids = torch.cat((input_ids, tok.view(-1, 1)), 1)       # model_factory.py:136-138
            attention_mask = torch.cat((attention_mask, torch.ones(B, 1, dtype=dt)), 1)
            first = False
        return input_ids


# ---------------------------------------------------------------------------------------
# conversions between the logical names and the reference's state_dict names (TP = 1)
# ---------------------------------------------------------------------------------------
def block_to_reference_state(bp, fused_qkv):
    """Logical block params -> names of the reference Block1D at tensor-parallel size 1.
    Fused layout is chunked k, v, q (attention.py:75)."""
    sd = {
        "norm1.module.weight": bp["norm1.weight"], "norm1.module.bias": bp["norm1.bias"],
        "norm2.module.weight": bp["norm2.weight"], "norm2.module.bias": bp["norm2.bias"],
        "attn.dense.weight": bp["dense.weight"], "attn.dense.bias": bp["dense.bias"],
        "mlp.dense_1.weight": bp["fc1.weight"], "mlp.dense_1.bias": bp["fc1.bias"],
        "mlp.dense_2.weight": bp["fc2.weight"], "mlp.dense_2.bias": bp["fc2.bias"],
    }
    if fused_qkv:
        sd["attn.query_key_value.weight"] = torch.cat([bp["k.weight"], bp["v.weight"], bp["q.weight"]], 0)
        sd["attn.query_key_value.bias"] = torch.cat([bp["k.bias"], bp["v.bias"], bp["q.bias"]], 0)
    else:
        for n, m in (("q", "query_"), ("k", "key_"), ("v", "value_")):
            sd[f"attn.{m}.weight"] = bp[f"{n}.weight"]
            sd[f"attn.{m}.bias"] = bp[f"{n}.bias"]
    return sd


def model_to_reference_state(params, depth, fused_qkv):
    """Logical model params -> reference PipelineModel state_dict names."""
    sd = {
        "embed.word_embeddings.weight": params["embed.word.weight"],
        "embed.position_embeddings.weight": params["embed.pos.weight"],
        "norm.module.weight": params["norm.weight"], "norm.module.bias": params["norm.bias"],
        "head.dense.weight": params["head.weight"],
    }
    for i in range(depth):
        pre = f"blocks.{i}."
        bp = {k[len(pre):]: v for k, v in params.items() if k.startswith(pre)}
        for k, v in block_to_reference_state(bp, fused_qkv).items():
            sd[pre + k] = v
    return sd
