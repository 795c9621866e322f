"""MultiHeadAttention1D with the reference's constructor and forward signature
(energonai/model/attention.py:9-60), built on one fused QKV GEMM that writes straight into
the key/value cache, the fused attention kernels, and a row-parallel output projection.

Differences a caller can observe, both deliberate:
  * generation steps (first_cache=False) return only the new position, [batch, 1, hidden];
    the reference returns the whole sequence by concatenating cached outputs
    (attention.py:129-135), whose earlier rows never change and are never consumed;
  * rows of left-padding queries are unspecified (the reference produces finite but
    meaningless values there, and nothing reads them).
"""
import torch
from torch import nn, dtype

from ..attention import attention_prefill, attention_decode
from ..gemm import gemm
from ..nn import Linear1D_Col, Linear1D_Row, FoldCache, tensor_version
from ..tp import get_tp, divide


class KVCache:
    """[batch, capacity, 3*local_hidden] buffer holding, per token, this rank's key | value |
    query projection (the reference caches the three projections too, attention.py:86-98,
    growing them with torch.cat).  `reserve` is the number of generation steps the caller
    announced: the prompt pass sizes the buffer for prompt + reserve positions, so that steps
    replayed from a captured graph (which cannot reallocate) always find room; appends are
    written in place by the QKV GEMM epilogue."""

    def __init__(self, reserve=256):
        self.buf, self.len, self.reserve = None, 0, reserve

    def capacity(self):
        return 0 if self.buf is None else self.buf.shape[1]

    def ensure(self, batch, need, width, dtype, device, exact=False):
        """Room for `need` positions (exact: allocate just that; else `reserve` more, so that
        eager appends do not reallocate every step).  Existing rows are kept."""
        if self.buf is not None and self.buf.shape[0] == batch and self.buf.shape[1] >= need and self.buf.dtype == dtype:
            return
        cap = need if exact else need + self.reserve
        new = torch.empty((batch, cap, width), dtype=dtype, device=device)
        if self.buf is not None and self.buf.shape[0] == batch and self.len > 0 and self.buf.dtype == dtype:
            new[:, :self.len] = self.buf[:, :self.len]
        self.buf = new

    def reset(self):
        self.len = 0


class MultiHeadAttention1D(nn.Module):
    def __init__(self,
                 hidden_size: int,
                 num_heads: int,
                 bias: bool = True,
                 dtype: dtype = torch.float16,
                 max_seq_len: int = 512,
                 fused_qkv: bool = True,
                 is_decoder: bool = True,
                 disable_past_cache=False) -> None:
        super().__init__()
        tp = get_tp()
        self.hidden_size = hidden_size
        self.attention_head_size = divide(hidden_size, num_heads)
        self.num_heads_local = divide(num_heads, tp.world_size)
        self.local_hidden = self.num_heads_local * self.attention_head_size
        self.fused_qkv, self.is_decoder, self.disable_past_cache = fused_qkv, is_decoder, disable_past_cache
        self.scaling = self.attention_head_size ** -0.5
        self.max_seq_len = max_seq_len
        if fused_qkv:
            # rows of this rank's shard are ordered key | value | query (attention.py:75)
            self.query_key_value = Linear1D_Col(hidden_size, 3 * hidden_size, bias=bias, dtype=dtype)
        else:
            self.query_ = Linear1D_Col(hidden_size, hidden_size, bias=bias, dtype=dtype)
            self.key_ = Linear1D_Col(hidden_size, hidden_size, bias=bias, dtype=dtype)
            self.value_ = Linear1D_Col(hidden_size, hidden_size, bias=bias, dtype=dtype)
        self.dense = Linear1D_Row(hidden_size, hidden_size, bias=True, dtype=dtype, parallel_input=True)
        self.past_cache = KVCache()
        self._packed_w = self._packed_b = None
        self._fold = FoldCache()

    # -- one [3*local_hidden, hidden] weight in k|v|q order, shared with the named parameters --
    def _packed(self):
        if self.fused_qkv:
            lin = self.query_key_value
            return lin.weight, lin.bias
        mods = (self.key_, self.value_, self.query_)
        hl = self.local_hidden
        ok = self._packed_w is not None and all(
            m.weight.data_ptr() == self._packed_w[i * hl:].data_ptr() for i, m in enumerate(mods))
        if not ok:
            with torch.no_grad():
                w = torch.cat([m.weight.detach() for m in mods], 0)
                b = torch.cat([m.bias.detach() for m in mods], 0) if mods[0].bias is not None else None
                for i, m in enumerate(mods):      # re-point the parameters at slices of the packed storage
                    m.weight.data = w[i * hl:(i + 1) * hl]
                    if b is not None:
                        m.bias.data = b[i * hl:(i + 1) * hl]
            self._packed_w, self._packed_b = w, b
        return self._packed_w, self._packed_b

    def _param_versions(self):
        mods = (self.query_key_value,) if self.fused_qkv else (self.key_, self.value_, self.query_)
        return tuple(tensor_version(t) for m in mods for t in (m.weight, m.bias) if t is not None)

    def forward(self, hidden_states, attention_mask=None, first_cache=False, seq_lens=None, residual=None,
                kv_state=None, fold_norm=None, transient_ok=False):
        """hidden_states [batch, seq, hidden].  attention_mask: additive, [batch, 1, 1, kv_len]
        (0 / -10000), or None.  With a cache, first_cache=True runs the whole prompt and any
        later call appends the last position.  `residual`, if given, is added to the output
        inside the projection's epilogue (the block's skip connection).  `kv_state`, used when a
        generation step is captured in a CUDA graph, is a device int32 pair [position, length]
        that the kernels read instead of host values; the cache must already have room.
        `fold_norm` (generation steps only): the LayerNorm1D in front of this module;
        hidden_states is then its un-normalised input and the QKV GEMM normalises on the fly.
        `transient_ok`: see Linear1D_Row.forward (the block consumes the result at once)."""
        B, S, _ = hidden_states.shape
        hl, d = self.local_hidden, self.attention_head_size
        w, b = self._packed()
        prefill = self.disable_past_cache or first_cache
        cache = self.past_cache
        if prefill:
            x = hidden_states.reshape(B * S, self.hidden_size)
            if self.disable_past_cache:
                buf = torch.empty((B, S, 3 * hl), dtype=x.dtype, device=x.device)
            else:
                cache.reset()
                # room for the announced generation steps too: a buffer kept from an earlier call
                # is reused only if it holds the whole of this one
                cache.ensure(B, S + max(0, cache.reserve), 3 * hl, x.dtype, x.device, exact=True)
                buf = cache.buf
            gemm(x, w, bias=b, static_weight=True, out=buf, out_rows_per_batch=S, out_batch_stride=buf.stride(0), out_ld=buf.stride(1))
            kv_len = S
            mask = attention_mask.reshape(B, -1) if attention_mask is not None else None
            ctx = attention_prefill(buf[:, :S, 2 * hl:], buf[:, :S, :hl], buf[:, :S, hl:2 * hl], d, mask=mask,
                                    causal=self.is_decoder, scale=self.scaling)
            if not self.disable_past_cache:
                cache.len = S
            res = residual
        else:
            x = hidden_states[:, -1, :]
            mask = attention_mask.reshape(B, -1) if attention_mask is not None else None
            fold = None
            if fold_norm is not None:
                w, colsum, bias32, eps = self._fold.get(w, b, fold_norm, self._param_versions())
                b, fold = None, (colsum, bias32, eps)
            if kv_state is None:
                pos = cache.len
                cache.ensure(B, pos + 1, 3 * hl, x.dtype, x.device)
                buf = cache.buf
                gemm(x, w, bias=b, static_weight=True, out=buf[:, pos:], out_rows_per_batch=1, out_batch_stride=buf.stride(0),
                     out_ld=buf.stride(1), ln_fold=fold)
                cache.len = kv_len = pos + 1
                ctx = attention_decode(buf[:, :, 2 * hl:], buf[:, :, :hl], buf[:, :, hl:2 * hl], d, kv_len, mask=mask,
                                       scale=self.scaling, q_in_cache=True)
            else:
                buf = cache.buf
                cap = buf.shape[1]
                if buf.shape[0] != B:
                    raise RuntimeError("attention: the cache was sized for another batch")
                gemm(x, w, bias=b, static_weight=True, out=buf, out_rows_per_batch=1, out_batch_stride=buf.stride(0), out_ld=buf.stride(1),
                     out_row_offset_device=kv_state[0:1], out_row_limit=cap, ln_fold=fold)
                ctx = attention_decode(buf[:, :, 2 * hl:], buf[:, :, :hl], buf[:, :, hl:2 * hl], d, cap, mask=mask,
                                       scale=self.scaling, q_in_cache=True, kv_len_device=kv_state[1:2])
            ctx = ctx.view(B, 1, hl)
            res = residual[:, -1:, :] if residual is not None else None
        return self.dense(ctx, residual=res, transient_ok=transient_ok)
