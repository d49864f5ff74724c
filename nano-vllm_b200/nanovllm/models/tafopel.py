"""Tafopel: a hybrid decoder whose layers are parallel blocks, ``x <- x + mixer(LN(x)) + ff(LN(x))``, with one weight-only
layer norm per block feeding both branches.  The mixer of a layer is latent attention (optionally borrowing an earlier
layer's key/value cache) or a Mamba-1 selective scan; the feed-forward is a gated dense block, a routed mixture of
experts with a shared expert, or absent.  config.json lists the layers and gives every size and constant.

The residual stream is fp32 in both number formats; projections, caches and branch outputs are bf16 (serving) or fp32.
Like the other models of this package it is a plain object: named device tensors and a flat list of launches per step,
the same for prompt portions, mixed batches and (captured in CUDA graphs) decode steps.

Cache and state: the model owns a paged cache per latent-attention layer that has its own key/value projection
(``[blocks * block_size, kv_rank + rot_dim]``, addressed through the engine's block tables and slot numbers) and one
state slot per live sequence for every selective-scan layer; the engine's block manager hands out both.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import mixops
from ..layers.latent_attention import LatentAttention
from ..layers.layernorm import ResidualLayerNorm
from ..layers.moe import GatedDenseFF, RoutedExpertsFF
from ..layers.selective_scan import SelectiveScanMixer
from ..utils.context import get_context

MIXERS = {"latent_attention": LatentAttention, "mamba1": SelectiveScanMixer}
DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


class TafopelConfig:
    """The parsed config.json plus the attribute names the engine reads from any model configuration."""
    architectures = ["Tafopel"]

    def __init__(self, raw: dict, max_position_embeddings: int = 1 << 20):
        self.raw = raw
        self.layers = raw["layers"]
        self.vocab_size = int(raw["vocab"])
        self.hidden_size = int(raw["width"])
        self.norm_eps = float(raw["norm"]["eps"])
        self.num_hidden_layers = len(self.layers)
        self.max_position_embeddings = int(raw.get("max_position", max_position_embeddings))
        self.eos_token_id = raw.get("eos")
        for i, layer in enumerate(self.layers):
            if layer["type"] not in MIXERS:
                raise ValueError(f"layer {i}: unknown mixer type {layer['type']!r}")
            src = layer["mixer"].get("kv_from")
            if src is not None:
                s = self.layers[src]
                if not (0 <= src < i) or s["type"] != "latent_attention" or s["mixer"].get("kv_from") is not None:
                    raise ValueError(f"layer {i}: kv_from must name an earlier latent-attention layer with its own cache")
                for key in ("kv_rank", "rot_dim", "rot"):
                    if s["mixer"][key] != layer["mixer"][key]:
                        raise ValueError(f"layer {i}: {key} differs from the layer whose cache it reads")


class _Block:
    __slots__ = ("norm", "mixer", "ff")


class TafopelForCausalLM:
    needs_block_tables = True        # attention always reads keys through the block tables, also in a first portion
    has_recurrent_state = True       # set per instance below
    supports_prefix_cache = False    # a cached prefix cannot be skipped: the recurrent state at its end is not kept

    def __init__(self, hf_config: TafopelConfig, tp_rank: int = 0, tp_size: int = 1, device="cuda", max_position: int | None = None,
                 dtype=torch.bfloat16):
        if tp_size != 1:
            raise NotImplementedError("Tafopel runs on one GPU (no tensor-parallel sharding of its mixers yet)")
        c = hf_config
        self.cfg, self.device, self.dtype = c, torch.device(device), dtype
        self.hidden, self.eps = c.hidden_size, c.norm_eps
        self.vocab_shard = c.vocab_size
        self.tp_rank, self.tp_size = tp_rank, tp_size
        max_position = int(max_position or c.max_position_embeddings)
        self.embed = torch.empty(c.vocab_size, self.hidden, dtype=dtype, device=self.device)
        self.lm_head = torch.empty(c.vocab_size, self.hidden, dtype=dtype, device=self.device)
        self.final_norm = ResidualLayerNorm(self.hidden, self.eps, dtype, self.device)
        self.blocks: list[_Block] = []
        tables: dict = {}
        for layer in c.layers:
            b = _Block()
            b.norm = ResidualLayerNorm(self.hidden, self.eps, dtype, self.device)
            if layer["type"] == "latent_attention":
                b.mixer = LatentAttention(self.hidden, layer["mixer"], self.eps, dtype, self.device, max_position)
                b.mixer.cos_sin = tables.setdefault(b.mixer.rot_key, b.mixer.cos_sin)       # layers with one rotation share its table
            else:
                b.mixer = SelectiveScanMixer(self.hidden, layer["mixer"], dtype, self.device)
            mlp = layer.get("mlp")
            if mlp is None:
                b.ff = None
            elif mlp["kind"] == "dense":
                b.ff = GatedDenseFF(self.hidden, mlp, dtype, self.device)
            elif mlp["kind"] == "moe":
                b.ff = RoutedExpertsFF(self.hidden, mlp, dtype, self.device)
            else:
                raise ValueError(f"unknown feed-forward kind {mlp['kind']!r}")
            self.blocks.append(b)
        self.has_recurrent_state = any(isinstance(b.mixer, SelectiveScanMixer) for b in self.blocks)
        self.block_size = 0
        self._bound = False
        self._mm_f32_out = True

    # ---- weights -----------------------------------------------------------------------------------------------------
    def load_hf_tensor(self, name: str, w: torch.Tensor) -> None:
        """Place one checkpoint tensor: ``embed``, ``head``, ``final.norm``, ``l<i>.norm1``, ``l<i>.mix.<leaf>``, ``l<i>.mlp.<leaf>``."""
        if name == "embed":
            self.embed.copy_(w); return
        if name == "head":
            self.lm_head.copy_(w); return
        if name == "final.norm":
            self.final_norm.weight.copy_(w); return
        head, _, rest = name.partition(".")
        if not (head.startswith("l") and head[1:].isdigit()) or int(head[1:]) >= len(self.blocks):
            raise KeyError(f"unexpected checkpoint tensor {name}")
        b = self.blocks[int(head[1:])]
        ok = False
        if rest == "norm1":
            b.norm.weight.copy_(w); ok = True
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
        for i, layer in enumerate(c.layers):
            p, m = f"l{i}.", layer["mixer"]
            out[p + "norm1"] = (W,)
            if layer["type"] == "latent_attention":
                H, d, rd, vd, R, Q = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
                out.update({p + "mix.dq": (Q, W), p + "mix.dq.norm": (Q,), p + "mix.uq": (H * (d + rd), Q), p + "mix.uk": (H * d, R),
                            p + "mix.uv": (H * vd, R), p + "mix.sink": (H,), p + "mix.o": (W, H * vd)})
                if m.get("kv_from") is None:
                    out.update({p + "mix.dkv": (R + rd, W), p + "mix.dkv.norm": (R,)})
            else:
                C, N, R, K = m["inner"], m["state"], m["dt_rank"], m["conv"]
                out.update({p + "mix.in": (2 * C, W), p + "mix.conv": (C, K), p + "mix.conv.b": (C,), p + "mix.x": (R + 2 * N, C),
                            p + "mix.dt": (C, R), p + "mix.dt.b": (C,), p + "mix.A_log": (C, N), p + "mix.D": (C,), p + "mix.o": (W, C)})
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if mlp["kind"] == "dense":
                out.update({p + "mlp.gate": (mlp["ff"], W), p + "mlp.up": (mlp["ff"], W), p + "mlp.down": (W, mlp["ff"])})
            else:
                for k in range(mlp["router"]["experts"]):
                    out[f"{p}mlp.e{k}.up"] = (mlp["expert"]["ff"], W)
                    out[f"{p}mlp.e{k}.down"] = (W, mlp["expert"]["ff"])
                out[p + "mlp.router"] = (mlp["router"]["experts"], W)
                if mlp.get("shared"):
                    s = mlp["shared"]["ff"]
                    out.update({p + "mlp.shared.up": (s, W), p + "mlp.shared.down": (W, s), p + "mlp.shared.sg": (1, W)})
        return out

    # ---- cache and state ---------------------------------------------------------------------------------------------
    def cache_block_bytes(self, block_size: int) -> int:
        elem = 4 if self.dtype == torch.float32 else 2
        return sum(b.mixer.cache_row_elems() for b in self.blocks if isinstance(b.mixer, LatentAttention)) * block_size * elem

    def state_slot_bytes(self) -> int:
        return sum(b.mixer.state_slot_bytes() for b in self.blocks if isinstance(b.mixer, SelectiveScanMixer))

    def bind_cache(self, num_blocks: int, block_size: int, num_state_slots: int) -> None:
        self.block_size = block_size
        for b in self.blocks:
            m = b.mixer
            if isinstance(m, LatentAttention):
                m.block_size = block_size
                if m.kv_from is None:
                    m.cache = torch.zeros(num_blocks * block_size, m.cache_row_elems(), dtype=self.dtype, device=self.device)
            else:
                m.bind_state(max(num_state_slots, 1))
        for b in self.blocks:
            m = b.mixer
            if isinstance(m, LatentAttention) and m.kv_from is not None:
                m.cache = self.blocks[m.kv_from].mixer.cache
        self._bound = True

    def unbind_cache(self) -> None:
        for b in self.blocks:
            m = b.mixer
            if isinstance(m, LatentAttention):
                m.cache = None
            else:
                m.conv_state = m.ssm_state = None
        self._bound = False

    def modules(self):
        return iter(())               # no paged-GQA attention operators: the cache is bound through bind_cache()

    # ---- forward ------------------------------------------------------------------------------------------------------
    @staticmethod
    def _spans(ctx, n: int) -> mixops.StepSpans:
        if ctx.is_prefill:
            return mixops.StepSpans(ctx.cu_seqlens_q.numel() - 1, int(ctx.max_seqlen_q), ctx.cu_seqlens_q, ctx.cu_seqlens_k, None)
        return mixops.StepSpans(n, 1, None, None, ctx.context_lens)

    @torch.inference_mode()
    def forward(self, input_ids: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        """-> the fp32 residual stream after the last layer, [tokens, width]."""
        if not self._bound:
            raise RuntimeError("bind_cache() first: this model has no cache-less path")
        ctx = get_context()
        spans = self._spans(ctx, input_ids.shape[0])
        x = mixops.embed(input_ids, self.embed)
        h = self.blocks[0].norm(x)
        last = len(self.blocks) - 1
        for i, b in enumerate(self.blocks):
            mix = b.mixer.forward(h, positions, ctx, spans)
            ff, ff32 = b.ff.forward(h) if b.ff is not None else (None, None)
            if i < last:
                h = self.blocks[i + 1].norm(x, a=mix, b=ff, b32=ff32)
            else:
                mixops.add_layernorm(x, None, self.eps, a=mix, b=ff, b32=ff32, norm=False)
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
        hn = self.final_norm(hidden, rows_idx=rows)
        if self.dtype == torch.float32:
            return F.linear(hn, self.lm_head)
        if self._mm_f32_out:
            try:
                return torch.mm(hn, self.lm_head.t(), out_dtype=torch.float32)        # bf16 operands, fp32 accumulator written as is
            except (RuntimeError, TypeError):
                self._mm_f32_out = False          # shapes or a library build without that output type: round once to bf16 instead
        return F.linear(hn, self.lm_head).float()
