"""Host-side pieces of the Tipetar integration (no GPU): configuration reader and registry, tensor names, the plain
implementation's own consistency, and replay bookkeeping without state slots."""
import json
import math

import pytest
import torch

import tipetar_helpers as th
from nanovllm.models import registry
from nanovllm.models.tipetar import TipetarConfig, TipetarForCausalLM
from oracle import tipetar_ref as ref


def test_registry_reads_the_architecture_key(tmp_path):
    cfg = th.config_a()
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    hf = registry.read_config(str(tmp_path))
    assert isinstance(hf, TipetarConfig) and hf.vocab_size == 97 and hf.num_hidden_layers == 4 and hf.hidden_size == 64
    assert hf.residual_mult == 0.6 and hf.norm_eps == 2e-5
    assert registry.model_class(hf).__name__ == "TipetarForCausalLM"


@pytest.mark.parametrize("bad", ["forward", "chain", "heads", "type", "kind", "groups"])
def test_config_rejects_what_the_design_does_not_have(bad):
    cfg = th.config_a()
    if bad == "forward":
        cfg["layers"][0]["mixer"]["kv_from"] = 2
    elif bad == "chain":
        cfg["layers"].append(dict(th.attn(kv_from=1), mlp=None))
    elif bad == "heads":
        cfg["layers"][3]["mixer"]["kv_heads"] = 4
    elif bad == "type":
        cfg["layers"][2]["type"] = "mamba1"
    elif bad == "kind":
        cfg["layers"][0]["mlp"]["kind"] = "dense"
    if bad == "groups":
        cfg["layers"][0]["mlp"]["router"]["groups"] = {"count": 3, "keep": 1}        # 8 router outputs do not split into 3 groups
        with pytest.raises(ValueError):
            TipetarForCausalLM(TipetarConfig(cfg), device="cpu")
        return
    with pytest.raises(ValueError):
        TipetarConfig(cfg)


@pytest.mark.parametrize("make", [th.config_a, th.config_b, th.config_c])
def test_tensor_names_and_loading(make):
    """Every checkpoint tensor has a place, nothing is left over, and a layer that reads another layer's keys has no key/value tensors."""
    cfg = make()
    model = TipetarForCausalLM(TipetarConfig(cfg), device="cpu")
    assert model.weight_shapes() == th.shapes(cfg)
    W = th.random_weights(cfg, 1)
    for k, v in W.items():
        model.load_hf_tensor(k, v)
    with pytest.raises(KeyError):
        model.load_hf_tensor("l0.mix.sink", torch.zeros(1))
    for i, layer in enumerate(cfg["layers"]):
        m = model.blocks[i].mixer
        if layer["mixer"].get("kv_from") is not None:
            assert m.cache_row_elems() == 0 and m.w_qkv.shape[0] == m.heads * m.dim
            with pytest.raises(KeyError):
                model.load_hf_tensor(f"l{i}.mix.k", torch.zeros(m.kv_heads * m.dim, cfg["width"]))
        else:
            assert torch.equal(m.w_qkv[m.q_cols:m.q_cols + m.k_cols], W[f"l{i}.mix.k"])
    assert model.cache_block_bytes(16) == sum(2 * 16 * l["mixer"]["kv_heads"] * (l["mixer"]["dim"] + l["mixer"]["vdim"])
                                              for l in cfg["layers"] if l["mixer"].get("kv_from") is None)
    assert not model.has_recurrent_state and model.state_slot_bytes() == 0


def test_distance_slopes():
    from nanovllm.layers.window_attention import distance_slopes
    for heads in (1, 3, 8, 20):
        s = distance_slopes(heads, "cpu")
        assert torch.allclose(s.double(), ref.slopes(heads), rtol=1e-7)
        assert abs(s[-1].item() - 2.0 ** -8) < 1e-9


def test_plain_attention_window_and_bias():
    """The plain implementation against a per-query loop written differently: explicit key ranges instead of a mask."""
    g = torch.Generator().manual_seed(0)
    H, G, d, vd, n, window = 4, 2, 6, 5, 40, 7
    q, k, v = (torch.randn(n, c, generator=g, dtype=torch.float64) for c in (H * d, G * d, G * vd))
    got = ref.windowed_attention(q, k, v, H, G, 0.3, window)
    for i in (0, 3, 6, 7, 39):
        for h in range(H):
            lo, grp = max(0, i - window + 1), h // 2
            s = torch.tensor([(q[i, h * d:(h + 1) * d] @ k[j, grp * d:(grp + 1) * d]).item() * 0.3 - 2.0 ** (-8 * (h + 1) / H) * (i - j)
                              for j in range(lo, i + 1)], dtype=torch.float64)
            p = torch.softmax(s, 0)
            want = sum(p[j - lo] * v[j, grp * vd:(grp + 1) * vd] for j in range(lo, i + 1))
            assert torch.allclose(got[i, h * vd:(h + 1) * vd], want, atol=1e-12)
    assert torch.equal(ref.visible(5, 0), torch.ones(5, 5).tril().bool())
    assert ref.visible(5, 2).sum().item() == 9


def test_plain_router_closed_groups_and_negative_scores():
    z = torch.tensor([[0.0, 0.0, 5.0, 0.0, 0.0, 0.0]], dtype=torch.float64)
    corr = torch.tensor([-5.0, -5.0, -9.0, -5.0, -5.5, -5.2], dtype=torch.float64)      # every choice score is negative
    # three groups of two; group scores: max(c0, c1), max(c2, c3), max(c4, c5); keep 1
    chosen, w = ref.route(z, corr, 2, 3, 1, 2.0)
    s = torch.softmax(z, -1)[0]
    c = s + corr
    best = max(range(3), key=lambda gi: max(c[2 * gi], c[2 * gi + 1]))
    assert sorted(chosen[0].tolist()) == [2 * best, 2 * best + 1]
    assert math.isclose(w.sum().item(), 2.0, rel_tol=1e-12)
    # the weight uses the score without the correction
    assert math.isclose((w[0, 0] / w[0, 1]).item(), (s[chosen[0, 0]] / s[chosen[0, 1]]).item(), rel_tol=1e-12)


def test_dictated_steps_without_state_slots():
    """A model without recurrent state runs dictated steps with zero state slots: pages are handed out, grown and taken back."""
    from nanovllm.config import Config
    from nanovllm.engine.scheduler import Scheduler
    from nanovllm.engine.sequence import Sequence
    hf = TipetarConfig(th.config_a())
    cfg = Config("unused", hf_config=hf, max_num_seqs=2, max_num_batched_tokens=64, max_model_len=64, kvcache_block_size=16,
                 num_kvcache_blocks=4, logits_only=True)
    cfg.num_state_slots, cfg.prefix_cache = 0, True
    Sequence.block_size = 16
    s = Scheduler(cfg)
    a, b = Sequence([1] * 20), Sequence([2] * 3)
    batch, varlen = s.plan_step([(a, [1] * 20), (b, [2] * 3)])
    assert varlen and len(a.block_table) == 2 and len(b.block_table) == 1
    s.postprocess_replay(batch)
    batch, varlen = s.plan_step([(a, [5]), (b, [6])])
    assert not varlen
    s.postprocess_replay(batch)
    s.retire(b)
    c = Sequence([3] * 30)
    batch, varlen = s.plan_step([(c, [3] * 30)])              # takes b's page and the last free one
    assert varlen and len(c.block_table) == 2
    with pytest.raises(RuntimeError):
        s.plan_step([(a, [1] * 30)])
