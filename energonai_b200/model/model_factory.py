"""PipelineModel and the model factories with the reference's interface
(energonai/model/model_factory.py:43-354), single pipeline stage.

The generation loop keeps the reference's contract (input_ids / attention_mask in, token ids
extended to max_tokens out; sampling through the same logits warpers; greedy = top_k 1) but
does the work once: the prompt is embedded and run through the blocks a single time, every
later step embeds and runs only the new token against the key/value caches, and the final
norm + LM head see only the last position (the reference re-embeds the whole sequence and
runs the head on every position each step, model_factory.py:112-131, with the same result for
the sampled token)."""
import os
from typing import Callable, Optional

import torch
from torch import dtype, nn

from ..nn import LayerNorm1D, can_fold
from .downstream import LMHead1D
from .embedding import Embedding1D
from .endecoder import Block1D
from .mlp import gelu_impl


class PipelineModel(nn.Module):
    def __init__(self,
                 vocab_size: int = 50257,
                 num_tokentypes: int = 0,
                 max_seq_len: int = 512,
                 hidden_size: int = 768,
                 num_heads: int = 12,
                 depth: int = 12,
                 mlp_ratio: float = 4.0,
                 layernorm_epsilon: float = 1e-5,
                 activation: Callable = gelu_impl,
                 padding_idx: int = 0,
                 dtype: dtype = torch.float16,
                 bias: bool = True,
                 apply_post_layernorm: bool = False,
                 first: bool = True,
                 last: bool = True,
                 fused_qkv: bool = True,
                 checkpoint: str = None,
                 model_name: str = None,
                 is_decoder: bool = True,
                 disable_past_cache=False,
                 vocab_parallel: bool = False) -> None:
        super().__init__()
        self.hidden_size, self.first, self.last = hidden_size, first, last
        self.max_seq_len, self.model_name = max_seq_len, model_name
        self.disable_past_cache = disable_past_cache
        self.eos_token_id = 50256          # the reference hard-codes this stop id (model_factory.py:133)
        self.use_cuda_graph = True         # greedy generation steps are captured once and replayed
        self.stop_check_every = 16         # replayed steps between two host reads of the stop condition
        # optional: generation steps run each layer as two launches (attention + one chained
        # kernel for the six GEMM / LayerNorm operations around it).  Off by default: measured on
        # OPT-13B, batch 16, the chained step is about 6 % slower than one kernel per operation
        # under programmatic dependent launch.
        self.use_decode_chain = os.environ.get("EB_CHAIN", "0") == "1"
        if first:
            self.embed = Embedding1D(hidden_size=hidden_size, vocab_size=vocab_size, max_seq_len=max_seq_len,
                                     num_tokentypes=num_tokentypes, padding_idx=padding_idx, dtype=dtype,
                                     vocab_parallel=vocab_parallel)
        self.blocks = nn.ModuleList()
        for id_ in range(depth):
            self.blocks.add_module(f'{id_}', Block1D(hidden_size=hidden_size, num_heads=num_heads, mlp_ratio=mlp_ratio,
                                                     activation=activation, layernorm_epsilon=layernorm_epsilon,
                                                     dtype=dtype, bias=bias, apply_post_layernorm=apply_post_layernorm,
                                                     max_seq_len=max_seq_len, fused_qkv=fused_qkv, is_decoder=is_decoder,
                                                     disable_past_cache=disable_past_cache))
        if last:
            self.norm = LayerNorm1D(normalized_shape=hidden_size, eps=layernorm_epsilon, dtype=dtype)
            self.head = LMHead1D(hidden_size=hidden_size, vocab_size=vocab_size, bias=False, dtype=dtype,
                                 vocab_parallel=vocab_parallel)

    def reserve_cache(self, new_tokens):
        """Size the key/value caches so `new_tokens` generation steps need no reallocation."""
        for blk in self.blocks:
            blk.attn.past_cache.reserve = max(1, int(new_tokens))

    # One generation step with every position-dependent quantity read from device memory, so
    # that the same sequence of launches can be captured once and replayed.
    def _chain_mode(self, batch_size, model_dtype):
        """How the generation step is launched: None = one kernel per operation (the default: on
        a tensor-parallel group the row-parallel GEMMs then carry their all-reduce in their own
        epilogue); "local" = per layer one attention kernel and one chained kernel for the six
        GEMM / LayerNorm operations around it; "exchange" = the same chain on a tensor-parallel
        group, with the two all-reduces of a layer carried inside it.  The chained forms are
        opt-in (EB_CHAIN=1 or use_decode_chain): measured on B200 with OPT-13B they lose, 7.8 ms
        per step against 6.5 ms on one GPU and 2.97 ms against 2.50 ms on the shard of an 8-way
        group, because the grid-wide hand-over between operations (arrival counter, polling,
        proxy fence) is slower than the hardware's own kernel boundary under programmatic
        dependent launch."""
        from ..tp import get_tp
        tp = get_tp()
        blk = self.blocks[0] if len(self.blocks) else None
        ok = (blk is not None and batch_size <= 128 and model_dtype in (torch.float16, torch.bfloat16)
              and not blk.apply_post_layernorm and not self.disable_past_cache and self.first and self.last)
        if not ok:
            return None
        if tp.world_size > 1:
            fits = tp.peer is not None and tp.peer.fits(batch_size, self.hidden_size)
            return "exchange" if fits and self.use_decode_chain else None
        return "local" if self.use_decode_chain else None

    def _build_chains(self, st):
        """The generation step as 1 + depth chained launches over fixed buffers:
        [norm1_0, qkv_0], then per layer, after its attention kernel,
        [out-proj + residual, norm2, FC1 + activation, FC2 + residual, norm1 / qkv of the next
        layer (or the final norm and the LM head)]  (energonai/model/endecoder.py:48-70,
        model_factory.py:124-131).  On a tensor-parallel group the two row-parallel products are
        exchanged and "+ bias + residual, LayerNorm" becomes the reduction that follows them."""
        from ..chain import Chain, gemm_op, layernorm_op, reduce_layernorm_op
        from ..tp import get_tp
        B = st["tok"].shape[0]
        dev, dt = st["tok"].device, st["add_mask"].dtype
        h = self.hidden_size
        f = self.blocks[0].mlp.dense_1.out_per_rank
        exchange = st["chain_mode"] == "exchange"
        comm = get_tp().peer if exchange else None
        new = lambda *shape, dtype=dt: torch.empty(shape, dtype=dtype, device=dev)
        xa, xb, x1, n, a = new(B, h), new(B, h), new(B, h), new(B, h), new(B, f)
        ctx = new(B, self.blocks[0].attn.local_hidden)
        logits = new(B, self.head.weight.shape[0], dtype=torch.float32)

        def norm_of(i):          # the LayerNorm in front of layer i's attention, or the model's final norm
            return self.norm if i == len(self.blocks) else self.blocks[i].norm1

        def proj_op(i):          # QKV of layer i into its cache row, or the LM head
            if i == len(self.blocks):
                return gemm_op(n, self.head.weight, logits, bias=self.head.dense.bias)
            blk = self.blocks[i]
            w, b = blk.attn._packed()
            buf = blk.attn.past_cache.buf
            return gemm_op(n, w, buf, bias=b, out_rows_per_batch=1, out_batch_stride=buf.stride(0), out_ld=buf.stride(1),
                           out_row_offset_device=st["kv_state"][0:1], out_row_limit=buf.shape[1])

        def ln_op(x, norm):
            return layernorm_op(x, n, norm.module.weight, norm.module.bias, norm.eps)

        groups = [[ln_op(xa, norm_of(0)), proj_op(0)]]
        x_in, x_out = xa, xb
        for i, blk in enumerate(self.blocks):
            nxt = norm_of(i + 1)
            if exchange:
                ops = [gemm_op(ctx, blk.attn.dense.weight, exchange=True),
                       reduce_layernorm_op(x1, h, bias=blk.attn.dense.bias, residual=x_in, y=n, gamma=blk.norm2.module.weight,
                                           beta=blk.norm2.module.bias, eps=blk.norm2.eps),
                       gemm_op(n, blk.mlp.dense_1.weight, a, bias=blk.mlp.dense_1.bias, act=blk.mlp.act_code),
                       gemm_op(a, blk.mlp.dense_2.weight, exchange=True),
                       reduce_layernorm_op(x_out, h, bias=blk.mlp.dense_2.bias, residual=x1, y=n, gamma=nxt.module.weight,
                                           beta=nxt.module.bias, eps=nxt.eps),
                       proj_op(i + 1)]
            else:
                ops = [gemm_op(ctx, blk.attn.dense.weight, x1, bias=blk.attn.dense.bias, residual=x_in),
                       ln_op(x1, blk.norm2),
                       gemm_op(n, blk.mlp.dense_1.weight, a, bias=blk.mlp.dense_1.bias, act=blk.mlp.act_code),
                       gemm_op(a, blk.mlp.dense_2.weight, x_out, bias=blk.mlp.dense_2.bias, residual=x1),
                       ln_op(x_out, nxt), proj_op(i + 1)]
            groups.append(ops)
            x_in, x_out = x_out, x_in
        nbytes = max(Chain.workspace_bytes(g, B, dev) for g in groups)
        ws = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
        st["chains"] = [Chain(g, B, dt, dev, workspace=ws, comm=comm) for g in groups]
        st["chain_bufs"] = {"x0": xa, "ctx": ctx, "logits": logits}

    def _chain_step(self, st):
        from ..attention import attention_decode
        if "chains" not in st:
            self._build_chains(st)
        bufs, chains = st["chain_bufs"], st["chains"]
        pos_long = st["kv_state"][0:1].to(torch.long)
        torch.add(self.embed.word_embeddings(st["tok"]), self.embed.position_embeddings(pos_long), out=bufs["x0"])
        chains[0].run()
        for i, blk in enumerate(self.blocks):
            at = blk.attn
            buf, hl = at.past_cache.buf, at.local_hidden
            attention_decode(buf[:, :, 2 * hl:], buf[:, :, :hl], buf[:, :, hl:2 * hl], at.attention_head_size, buf.shape[1],
                             mask=st["add_mask"], scale=at.scaling, q_in_cache=True, kv_len_device=st["kv_state"][1:2],
                             out=bufs["ctx"])
            chains[i + 1].run()
        logits = bufs["logits"]
        if self.head.vocab_parallel:
            from ..tp import get_tp
            logits = get_tp().all_gather_last_dim(logits)
        return logits

    def _static_step(self, st):
        if st.get("chain_mode"):
            tok = self._chain_step(st).argmax(-1)
            st["out_ids"].index_copy_(1, st["kv_state"][1:2].to(torch.long), tok.view(-1, 1))
            st["tok"].copy_(tok)
            st["kv_state"].add_(1)
            return
        fused = st.get("hidden") is not None
        if fused:
            hidden = st["hidden"]               # the new token's embedding, left there by the previous step's tail
        else:
            pos_long = st["kv_state"][0:1].to(torch.long)
            hidden = self.embed.word_embeddings(st["tok"].view(-1, 1)) + self.embed.position_embeddings(pos_long).unsqueeze(0)
        for block in self.blocks:
            hidden = block(hidden_states=hidden, attention_mask=st["mask4"], first_cache=False, kv_state=st["kv_state"])
        logits = self._last_logits(hidden)
        if fused:
            # one launch: arg-max, the token into its column, its embedding for the next step, positions advanced
            from ..step import greedy_step
            from ..tp import get_tp
            we = self.embed.word_embeddings
            split = getattr(we, "vocab_start", None) is not None
            greedy_step(logits, st["out_ids"], st["tok"], st["kv_state"], st["step_counter"], word_emb=we.weight,
                        pos_emb=self.embed.position_embeddings.weight, hidden_out=st["hidden"].view(-1, self.hidden_size),
                        vocab_start=we.vocab_start if split else 0, add_pos=(not split) or get_tp().rank == 0)
            if split:
                get_tp().all_reduce(st["hidden"])
            return
        tok = logits.argmax(-1)
        st["out_ids"].index_copy_(1, st["kv_state"][1:2].to(torch.long), tok.view(-1, 1))   # the new token's index
        st["tok"].copy_(tok)
        st["kv_state"].add_(1)

    def _last_logits(self, hidden, record=None):
        """Final norm + LM head of a generation step, hidden [batch, 1, hidden_size]."""
        fold = len(self.blocks) > 0 and self.blocks[0].fold_layernorm
        if record is None and can_fold(hidden.shape[0], hidden.dtype, fold):
            return self.head(hidden, fold_norm=self.norm)[:, -1, :]
        last_hidden = self.norm(hidden)
        if record is not None:
            record.setdefault("hidden", []).append(last_hidden[:, -1, :].clone())
        return self.head(last_hidden)[:, -1, :]

    def _graph_state(self, batch_size, tgt_len, model_dtype, dev, ids_dtype):
        key = (batch_size, tgt_len, model_dtype, ids_dtype, tuple(b.attn.past_cache.buf.data_ptr() for b in self.blocks))
        st = getattr(self, "_decode_state", None)
        if st is None or st["key"] != key:
            add_mask = torch.zeros((batch_size, tgt_len), dtype=model_dtype, device=dev)
            st = {"key": key, "graph": None, "add_mask": add_mask, "mask4": add_mask.view(batch_size, 1, 1, tgt_len),
                  "out_ids": torch.empty((batch_size, tgt_len), dtype=ids_dtype, device=dev),
                  "tok": torch.empty((batch_size,), dtype=ids_dtype, device=dev),
                  "kv_state": torch.zeros(2, dtype=torch.int32, device=dev),
                  "chain_mode": self._chain_mode(batch_size, model_dtype)}
            # the step's tail as one launch (eb_greedy_step) needs int64 ids, no token-type table
            # and logits of the embedding's dtype; otherwise the framework's kernels do it
            if (st["chain_mode"] is None and ids_dtype == torch.int64 and self.embed.tokentype_embeddings is None
                    and self.embed.position_embeddings.weight.dtype == model_dtype
                    and os.environ.get("EB_FUSED_TAIL", "1") != "0"):
                st["hidden"] = torch.empty((batch_size, 1, self.hidden_size), dtype=model_dtype, device=dev)
                st["step_counter"] = torch.zeros(1, dtype=torch.int32, device=dev)
            self._decode_state = st
        return st

    @torch.inference_mode()
    def forward(self, hidden_states=None, input_ids=None, attention_mask=None, seq_lens=None,
                max_tokens: Optional[int] = None, top_k: Optional[int] = None, top_p: Optional[float] = None,
                temperature: Optional[float] = None, record=None):
        batch_size, cur_len = input_ids.shape
        tgt_len = cur_len + 1 if not max_tokens else max_tokens
        if cur_len >= tgt_len:
            return input_ids
        if attention_mask is None:
            attention_mask = torch.ones_like(input_ids)
        dev = input_ids.device
        model_dtype = self.norm.module.weight.dtype
        self.reserve_cache(tgt_len - cur_len)
        greedy = top_k == 1 and (temperature is None or temperature > 0)
        step_times = record.setdefault("step_events", []) if record is not None else None
        from .. import _lib
        launches0, replayed = _lib.launch_count, 0

        def mark():
            if step_times is not None:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                step_times.append(ev)

        # ---- prompt pass ----
        add_mask_prompt = (1.0 - attention_mask.view(batch_size, -1).to(model_dtype)) * -10000.0
        mark()
        hidden_states = self.embed(input_ids)
        mask4 = add_mask_prompt.view(batch_size, 1, 1, cur_len)
        for block in self.blocks:
            hidden_states = block(hidden_states=hidden_states, attention_mask=mask4, first_cache=True)
        last_hidden = self.norm(hidden_states[:, -1:, :].contiguous())
        logits = self.head(last_hidden)[:, -1, :]
        if record is not None:
            record.setdefault("logits", []).append(logits.clone())
            record.setdefault("hidden", []).append(last_hidden[:, -1, :].clone())
        tok = logits.argmax(-1) if greedy else self.generate(input_ids, logits, top_k=top_k, top_p=top_p,
                                                             temperature=temperature)
        mark()
        if not max_tokens:
            return tok
        if torch.all(tok == self.eos_token_id):
            return input_ids

        # ---- generation steps ----
        for blk in self.blocks:
            # steps driven by device-side positions cannot grow the cache: it must hold the whole call
            if not self.disable_past_cache and blk.attn.past_cache.capacity() < tgt_len:
                raise RuntimeError(f"key/value cache holds {blk.attn.past_cache.capacity()} positions, {tgt_len} needed")
        st = self._graph_state(batch_size, tgt_len, model_dtype, dev, input_ids.dtype)
        st["add_mask"].zero_()
        st["add_mask"][:, :cur_len] = add_mask_prompt
        out_ids = st["out_ids"]
        out_ids[:, :cur_len] = input_ids
        out_ids[:, cur_len] = tok
        st["tok"].copy_(tok)
        st["kv_state"].copy_(torch.tensor([cur_len, cur_len + 1], dtype=torch.int32), non_blocking=False)
        if st.get("hidden") is not None:    # the first generated token's embedding; later ones come from the step's tail
            st["hidden"].copy_(self.embed(tok.view(-1, 1), past_key_values_length=cur_len))
        use_graph = greedy and self.use_cuda_graph and (record is None or record.get("allow_graph", False))
        produced = cur_len + 1
        checked = cur_len + 1                                  # columns of out_ids already tested for the stop condition
        for pos in range(cur_len + 1, tgt_len):
            if use_graph:
                if st["graph"] is None and pos == cur_len + 1:
                    before = _lib.launch_count
                    self._static_step(st)                      # eager once: also warms every kernel up
                    st["launches"] = _lib.launch_count - before
                elif st["graph"] is None:
                    g = torch.cuda.CUDAGraph()
                    before = _lib.launch_count
                    with torch.cuda.graph(g):
                        self._static_step(st)
                    launches0 += _lib.launch_count - before    # captured, not executed
                    st["graph"] = g
                    g.replay()
                    replayed += st["launches"]
                else:
                    st["graph"].replay()
                    replayed += st["launches"]
                mark()
                # The reference stops when every sequence has just produced the stop token
                # (model_factory.py:133-134).  Asking after every step would make the host wait for
                # the device once per token; replays are queued ahead instead and the question is
                # asked for a window of steps at a time.  Steps queued beyond the stopping point
                # only wrote cache rows and columns that are cut off below.
                if (pos - cur_len) % self.stop_check_every == 0 or pos == tgt_len - 1:
                    hit = (out_ids[:, checked:pos + 1] == self.eos_token_id).all(0).nonzero()
                    if hit.numel():
                        produced = checked + int(hit[0])
                        break
                    checked = pos + 1
                produced = pos + 1
                continue
            hidden_states = self.embed(tok.view(-1, 1), past_key_values_length=pos - 1)
            mask4 = st["add_mask"][:, :pos].view(batch_size, 1, 1, pos)
            for block in self.blocks:
                hidden_states = block(hidden_states=hidden_states, attention_mask=mask4, first_cache=False)
            logits = self._last_logits(hidden_states, record)
            if record is not None:
                record.setdefault("logits", []).append(logits.clone())
            tok = logits.argmax(-1) if greedy else self.generate(out_ids[:, :pos], logits, top_k=top_k, top_p=top_p,
                                                                 temperature=temperature)
            out_ids[:, pos] = tok
            mark()
            if torch.all(tok == self.eos_token_id):
                break
            produced = pos + 1
        for blk in self.blocks:                                # host bookkeeping of the cache length
            blk.attn.past_cache.len = produced - 1
        self.launches_last_call = _lib.launch_count - launches0 + replayed   # kernels of this library executed
        return out_ids[:, :produced].clone()

    def get_logits_processor(self, top_k=None, top_p=None, temperature=None):
        from transformers.generation import (LogitsProcessorList, TemperatureLogitsWarper, TopKLogitsWarper,
                                             TopPLogitsWarper)
        processor_list = LogitsProcessorList()
        if temperature is not None and temperature != 1.0:
            processor_list.append(TemperatureLogitsWarper(temperature))
        if top_k is not None and top_k != 0:
            processor_list.append(TopKLogitsWarper(top_k))
        if top_p is not None and top_p < 1.0:
            processor_list.append(TopPLogitsWarper(top_p))
        return processor_list

    def generate(self, input_ids, logits, top_k=None, top_p=None, temperature=None):
        """model_factory.py:153-159 on last-position logits [batch, vocab]."""
        logits = self.get_logits_processor(top_k, top_p, temperature)(input_ids, logits)
        probs = torch.softmax(logits, -1, dtype=torch.float)
        return torch.multinomial(probs, num_samples=1).squeeze(1)


def create_pipeline_model(depth: int = 48, layer_partitions=None, **model_kwargs):
    """Single-stage version of model_factory.py:182-226 (pipeline parallelism is outside the
    tensor-parallel layer path this package implements)."""
    if layer_partitions is not None:
        raise RuntimeError("pipeline partitioning is not supported; run with one pipeline stage")
    model_kwargs = dict(model_kwargs)
    model_kwargs.update(first=True, last=True, depth=depth)
    model = PipelineModel(**model_kwargs)
    model = model.cuda() if torch.cuda.is_available() else model
    # model_factory.py:212-224: a checkpoint is loaded only when the model family is named
    if model_kwargs.get("checkpoint") and model_kwargs.get("model_name"):
        from ..utils import load_175b, load_checkpoint, processing_HF_GPT, processing_OPT
        if not os.path.exists(model_kwargs["checkpoint"]):
            raise FileNotFoundError(f"checkpoint {model_kwargs['checkpoint']} not found")
        if model_kwargs["model_name"] == "opt-175b":
            load_175b(model_kwargs["checkpoint"], model)
        else:
            preprocess_fn = {"hf_gpt2": processing_HF_GPT, "opt": processing_OPT}.get(model_kwargs["model_name"])
            extra = {k: v for k, v in model_kwargs.items() if k == "prefix"}
            load_checkpoint(model_kwargs["checkpoint"], model, preprocess_fn=preprocess_fn, **extra)
    return model


def _opt(hidden, depth, heads, **kwargs):
    model_kwargs = dict(vocab_size=50272, hidden_size=hidden, depth=depth, max_seq_len=2050, num_heads=heads,
                        activation=nn.functional.relu, is_decoder=True, fused_qkv=False, model_name="opt",
                        disable_past_cache=False)
    model_kwargs.update(kwargs)
    return create_pipeline_model(**model_kwargs)


def opt_125M(**kwargs):
    return _opt(768, 12, 12, **kwargs)


def opt_6B(**kwargs):
    return _opt(4096, 32, 32, **kwargs)


def opt_13B(**kwargs):
    """OPT-13B shape (40 layers, hidden 5120, 40 heads); the reference has no factory of this
    name, the shape follows its opt_* pattern (model_factory.py:281-339)."""
    return _opt(5120, 40, 40, **kwargs)


def opt_30B(**kwargs):
    return _opt(7168, 48, 56, **kwargs)


def opt_66B(**kwargs):
    return _opt(9216, 64, 72, **kwargs)


def opt_175B(**kwargs):
    return _opt(12288, 96, 96, **dict(dict(fused_qkv=True, model_name="opt-175b"), **kwargs))


def gpt2_small(**kwargs):
    return create_pipeline_model(**dict(dict(hidden_size=768, depth=12, num_heads=12, is_decoder=True), **kwargs))


def gpt2_large(**kwargs):
    return create_pipeline_model(**dict(dict(hidden_size=1536, depth=36, num_heads=12, is_decoder=True), **kwargs))


def gpt2_8B(**kwargs):
    return create_pipeline_model(**dict(dict(hidden_size=3072, depth=72, num_heads=24, is_decoder=True), **kwargs))


def gpt3(**kwargs):
    return create_pipeline_model(**dict(dict(hidden_size=12288, depth=12, num_heads=96, is_decoder=True), **kwargs))


def hf_gpt2(**kwargs):
    return create_pipeline_model(**dict(dict(hidden_size=768, depth=12, max_seq_len=1024, num_heads=12, fused_qkv=False,
                                             model_name="hf_gpt2", is_decoder=True), **kwargs))


def bert_small(**kwargs):
    return create_pipeline_model(**dict(dict(hidden_size=768, depth=12, num_heads=12, is_decoder=False), **kwargs))


def bert_large(**kwargs):
    return create_pipeline_model(**dict(dict(hidden_size=1024, depth=24, num_heads=16, is_decoder=False), **kwargs))


def bert_8B(**kwargs):
    return create_pipeline_model(**dict(dict(hidden_size=3072, depth=72, num_heads=24, is_decoder=False), **kwargs))


def bert_175B(**kwargs):
    return create_pipeline_model(**dict(dict(hidden_size=12288, depth=96, num_heads=96, is_decoder=False), **kwargs))
