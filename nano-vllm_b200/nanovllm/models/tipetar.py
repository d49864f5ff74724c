"""Tipetar: a decoder whose layers put the norm on each sublayer's OUTPUT and scale the residual update,
``x <- x + m * norm1(mixer(x))``, then ``x <- x + m * norm2(ff(x))`` (the sublayers read the stream itself).  The mixer is
grouped-query attention with a sliding window, a linear distance bias and no rotation, its queries and keys normalised over
the whole projection; a layer may read an earlier layer's keys and values instead of projecting its own.  The feed-forward
is a group-routed mixture of gated experts with a softmax router, a choice correction, identity experts and a shared
expert, or absent.  config.json (``"architecture": "Tipetar"``) lists the layers and gives every size and constant.

The residual stream is fp32 in both number formats; projections, caches and branch outputs are bf16 (serving) or fp32.
Like the other models of this package it is a plain object: named device tensors and a flat list of launches per step,
the same for prompt portions, mixed batches and (captured in CUDA graphs) decode steps.

Cache: one paged key/value cache per attention layer that owns a key/value projection
(``[blocks * block_size, kv_heads * (dim + vdim)]``, addressed through the engine's block tables and slot numbers).
There is no recurrent state, so a cached prefix can be skipped like in any attention-only decoder.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import mixops
from ..layers.layernorm import SublayerOutputNorm
from ..layers.moe import GroupRoutedExpertsFF
from ..layers.window_attention import BiasedWindowAttention
from ..utils.context import get_context


class TipetarConfig:
    """The parsed config.json plus the attribute names the engine reads from any model configuration."""
    architectures = ["Tipetar"]

    def __init__(self, raw: dict, max_position_embeddings: int = 1 << 20):
        self.raw = raw
        self.layers = raw["layers"]
        self.vocab_size = int(raw["vocab"])
        self.hidden_size = int(raw["width"])
        self.norm_eps = float(raw["norm"]["eps"])
        self.residual_mult = float(raw.get("residual_mult", 1.0))
        self.num_hidden_layers = len(self.layers)
        self.max_position_embeddings = int(raw.get("max_position", max_position_embeddings))
        self.eos_token_id = raw.get("eos")
        for i, layer in enumerate(self.layers):
            if layer["type"] != "attention":
                raise ValueError(f"layer {i}: unknown mixer type {layer['type']!r}")
            mlp = layer.get("mlp")
            if mlp is not None and mlp.get("kind") != "moe":
                raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
            src = layer["mixer"].get("kv_from")
            if src is not None:
                if not (0 <= src < i) or self.layers[src]["mixer"].get("kv_from") is not None:
                    raise ValueError(f"layer {i}: kv_from must name an earlier layer with a key/value projection of its own")
                for key in ("kv_heads", "dim", "vdim"):
                    if self.layers[src]["mixer"][key] != layer["mixer"][key]:
                        raise ValueError(f"layer {i}: {key} differs from the layer whose keys and values it reads")


class _Block:
    __slots__ = ("mixer", "norm1", "ff", "norm2")


class TipetarForCausalLM:
    needs_block_tables = True        # attention always reads keys through the block tables, also in a first portion
    has_recurrent_state = False
    supports_prefix_cache = True

    def __init__(self, hf_config: TipetarConfig, tp_rank: int = 0, tp_size: int = 1, device="cuda", max_position: int | None = None,
                 dtype=torch.bfloat16):
        if tp_size != 1:
            raise NotImplementedError("Tipetar runs on one GPU (no tensor-parallel sharding of its mixers yet)")
        c = hf_config
        self.cfg, self.device, self.dtype = c, torch.device(device), dtype
        self.hidden, self.eps, self.mult = c.hidden_size, c.norm_eps, c.residual_mult
        self.vocab_shard = c.vocab_size
        self.tp_rank, self.tp_size = tp_rank, tp_size
        self.embed = torch.empty(c.vocab_size, self.hidden, dtype=dtype, device=self.device)
        self.lm_head = torch.empty(c.vocab_size, self.hidden, dtype=dtype, device=self.device)
        self.final_norm = torch.zeros(self.hidden, dtype=dtype, device=self.device)
        self.blocks: list[_Block] = []
        for layer in c.layers:
            b = _Block()
            b.mixer = BiasedWindowAttention(self.hidden, layer["mixer"], self.eps, dtype, self.device)
            b.norm1 = SublayerOutputNorm(self.hidden, self.eps, dtype, self.device)
            mlp = layer.get("mlp")
            b.ff = GroupRoutedExpertsFF(self.hidden, mlp, dtype, self.device) if mlp is not None else None
            b.norm2 = SublayerOutputNorm(self.hidden, self.eps, dtype, self.device) if mlp is not None else None
            self.blocks.append(b)
        self.block_size = 0
        self._bound = False
        self._mm_f32_out = True

    # ---- weights -----------------------------------------------------------------------------------------------------
    def load_hf_tensor(self, name: str, w: torch.Tensor) -> None:
        """Place one checkpoint tensor: ``embed``, ``head``, ``final.norm``, ``l<i>.norm1|norm2``, ``l<i>.mix.<leaf>``, ``l<i>.mlp.<leaf>``."""
        if name == "embed":
            self.embed.copy_(w); return
        if name == "head":
            self.lm_head.copy_(w); return
        if name == "final.norm":
            self.final_norm.copy_(w); return
        head, _, rest = name.partition(".")
        if not (head.startswith("l") and head[1:].isdigit()) or int(head[1:]) >= len(self.blocks):
            raise KeyError(f"unexpected checkpoint tensor {name}")
        b = self.blocks[int(head[1:])]
        ok = False
        if rest == "norm1":
            b.norm1.weight.copy_(w); ok = True
        elif rest == "norm2" and b.norm2 is not None:
            b.norm2.weight.copy_(w); ok = True
        elif rest.startswith("mix."):
            ok = b.mixer.load(rest[4:], w)
        elif rest.startswith("mlp.") and b.ff is not None:
            ok = b.ff.load(rest[4:], w)
        if not ok:
            raise KeyError(f"unexpected checkpoint tensor {name}")

    def weight_shapes(self) -> dict:
        """name -> shape of every checkpoint tensor of this configuration (random initialisation, tests)."""
        c, W = self.cfg, self.hidden
        out = {"embed": (c.vocab_size, W), "head": (c.vocab_size, W), "final.norm": (W,)}
        for i, b in enumerate(self.blocks):
            p = f"l{i}."
            out[p + "norm1"] = (W,)
            out.update({p + "mix." + k: v for k, v in b.mixer.weight_shapes(W).items()})
            if b.ff is not None:
                out[p + "norm2"] = (W,)
                out.update({p + "mlp." + k: v for k, v in b.ff.weight_shapes(W).items()})
        return out

    zero_centred = ("norm1", "norm2", "final.norm", "correction")      # 1-D tensors whose neutral value is 0, not 1 (random initialisation)

    # ---- cache ---------------------------------------------------------------------------------------------------------
    def cache_block_bytes(self, block_size: int) -> int:
        elem = 4 if self.dtype == torch.float32 else 2
        return sum(b.mixer.cache_row_elems() for b in self.blocks) * block_size * elem

    def state_slot_bytes(self) -> int:
        return 0

    def bind_cache(self, num_blocks: int, block_size: int, num_state_slots: int = 0) -> None:
        self.block_size = block_size
        for b in self.blocks:
            m = b.mixer
            m.block_size = block_size
            if m.kv_from is None:
                m.cache = torch.zeros(num_blocks * block_size, m.cache_row_elems(), dtype=self.dtype, device=self.device)
        for b in self.blocks:
            if b.mixer.kv_from is not None:
                b.mixer.cache = self.blocks[b.mixer.kv_from].mixer.cache
        self._bound = True

    def unbind_cache(self) -> None:
        for b in self.blocks:
            b.mixer.cache = None
        self._bound = False

    def modules(self):
        return iter(())               # no paged-GQA attention operators of the first library: the cache is bound through bind_cache()

    # ---- forward ------------------------------------------------------------------------------------------------------
    @staticmethod
    def _spans(ctx, n: int) -> mixops.StepSpans:
        if ctx.is_prefill:
            return mixops.StepSpans(ctx.cu_seqlens_q.numel() - 1, int(ctx.max_seqlen_q), ctx.cu_seqlens_q, ctx.cu_seqlens_k, None)
        return mixops.StepSpans(n, 1, None, None, ctx.context_lens)

    @torch.inference_mode()
    def forward(self, input_ids: torch.Tensor, positions: torch.Tensor, taps: list | None = None) -> torch.Tensor:
        """-> the fp32 residual stream after the last layer, [tokens, width].  ``taps`` (a list) collects a copy of the
        stream after every layer."""
        if not self._bound:
            raise RuntimeError("bind_cache() first: this model has no cache-less path")
        ctx = get_context()
        n = input_ids.shape[0]
        spans = self._spans(ctx, n)
        half = self.dtype != torch.float32
        h = torch.empty(n, self.hidden, dtype=self.dtype, device=self.device) if half else None
        x = mixops.embed(input_ids, self.embed, copy=h)
        if not half:
            h = x                                           # 32-bit format: the sublayers read the stream in place
        for b in self.blocks:
            b.norm1(x, b.mixer.forward(h, ctx, spans), self.mult, copy=h if half else None)
            if b.ff is not None:
                b.norm2(x, b.ff.forward(h, x), self.mult, copy=h if half else None)
            if taps is not None:
                taps.append(x.clone())
        return x

    __call__ = forward

    @torch.inference_mode()
    def last_token_rows(self, hidden: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError("the fused LM head takes bf16 rows; this model normalises selected rows in compute_logits")

    @torch.inference_mode()
    def compute_logits(self, hidden: torch.Tensor) -> torch.Tensor:
        """fp32 logits of the step's last token per sequence, or of the rows named by ``ctx.logit_rows`` (int32)."""
        ctx = get_context()
        rows = getattr(ctx, "logit_rows", None)
        if rows is None and ctx.is_prefill:
            rows = (ctx.cu_seqlens_q[1:] - 1).to(torch.int32)
        hn = mixops.rmsnorm_rows(hidden, self.final_norm, self.eps, w_offset=1.0, rows_idx=rows)
        if self.dtype == torch.float32:
            return F.linear(hn, self.lm_head)
        if self._mm_f32_out:
            try:
                return torch.mm(hn, self.lm_head.t(), out_dtype=torch.float32)        # bf16 operands, fp32 accumulator written as is
            except (RuntimeError, TypeError):
                self._mm_f32_out = False          # shapes or a library build without that output type: round once to bf16 instead
        return F.linear(hn, self.lm_head).float()
