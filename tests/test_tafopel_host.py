"""Host-side pieces of the Tafopel integration (no GPU): configuration reader and registry, rotary table, state slots and
replay bookkeeping in the block manager and scheduler, and the plain implementation's own consistency."""
import json
import os

import pytest
import torch

import tafopel_helpers as th
from nanovllm.config import Config
from nanovllm.engine.block_manager import BlockManager
from nanovllm.engine.scheduler import Scheduler
from nanovllm.engine.sequence import Sequence
from nanovllm.layers.rotary_embedding import build_interleaved_cos_sin
from nanovllm.models import registry
from nanovllm.models.tafopel import TafopelConfig
from oracle import tafopel_ref as ref


def test_registry_reads_the_architecture_key(tmp_path):
    cfg = th.config_a()
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    hf = registry.read_config(str(tmp_path))
    assert isinstance(hf, TafopelConfig) and hf.vocab_size == 97 and hf.num_hidden_layers == 4 and hf.hidden_size == 64
    assert registry.model_class(hf).__name__ == "TafopelForCausalLM"
    (tmp_path / "config.json").write_text(json.dumps(dict(cfg, architecture="Nope")))
    with pytest.raises(ValueError):
        registry.read_config(str(tmp_path))


@pytest.mark.parametrize("bad", ["forward", "chain", "rank", "type"])
def test_config_rejects_bad_cache_borrowing(bad):
    cfg = th.config_a()
    if bad == "forward":
        cfg["layers"][1]["mixer"]["kv_from"] = 3
    elif bad == "chain":
        cfg["layers"].append(dict(th.latent(kv_from=3), mlp=None))
    elif bad == "rank":
        cfg["layers"][3]["mixer"]["kv_rank"] = 48
    else:
        cfg["layers"][3]["mixer"]["kv_from"] = 0
    with pytest.raises(ValueError):
        TafopelConfig(cfg)


@pytest.mark.parametrize("scaling", [True, False])
def test_rotary_table_matches_plain_implementation(scaling):
    r = th.rot(12, 5000.0, scaling)
    table = build_interleaved_cos_sin(12, 300, 5000.0, r.get("scaling"))
    cos, sin = ref.rotary_tables(r, 300)
    assert table.shape == (300, 12)
    assert torch.allclose(table[:, :6].double(), cos, atol=1e-7) and torch.allclose(table[:, 6:].double(), sin, atol=1e-7)
    if scaling:         # interpolation changes the slow pairs only, and scales the magnitude
        plain = build_interleaved_cos_sin(12, 300, 5000.0, None)
        assert not torch.allclose(table, plain)
        assert abs(table[0, 0].item() - (0.1 * torch.log(torch.tensor(4.0)).item() + 1.0)) < 1e-6


def test_shapes_beyond_the_kernels_are_refused_at_construction():
    from nanovllm.layers.latent_attention import LatentAttention
    from nanovllm.layers.selective_scan import SelectiveScanMixer
    with pytest.raises(ValueError, match="kv_rank"):
        LatentAttention(64, th.latent(kv_rank=520)["mixer"], 1e-5, torch.float32, "cpu", 16)
    with pytest.raises(ValueError, match="state"):
        SelectiveScanMixer(64, th.mamba(state=129)["mixer"], torch.float32, "cpu")
    LatentAttention(64, th.latent(kv_rank=512)["mixer"], 1e-5, torch.float32, "cpu", 16)
    SelectiveScanMixer(64, th.mamba(state=128)["mixer"], torch.float32, "cpu")


def test_state_slots_follow_the_blocks():
    bm = BlockManager(6, 4, num_state_slots=2, prefix_cache=False)
    Sequence.block_size = 4
    a, b, c = Sequence(list(range(7))), Sequence(list(range(5))), Sequence([1])
    assert bm.can_allocate(a) == 0
    bm.allocate(a, 0)
    bm.allocate(b, 0)
    assert (a.state_slot, b.state_slot) == (0, 1) and len(a.block_table) == 2 and len(b.block_table) == 2
    assert bm.can_allocate(c) == -1                      # blocks are free, slots are not
    bm.deallocate(a)
    assert a.state_slot == -1 and bm.can_allocate(c) == 0
    bm.allocate(c, 0)
    assert c.state_slot == 0                             # the slot (and a's first page) change hands
    assert c.block_table[0] not in b.block_table


def test_no_block_is_shared_without_a_prefix_cache():
    bm = BlockManager(8, 4, num_state_slots=4, prefix_cache=False)
    Sequence.block_size = 4
    a, b = Sequence(list(range(9))), Sequence(list(range(9)))
    bm.allocate(a, bm.can_allocate(a))
    a.num_scheduled_tokens = 9
    bm.hash_blocks(a)
    assert bm.can_allocate(b) == 0
    bm.allocate(b, 0)
    assert not set(a.block_table) & set(b.block_table) and b.num_cached_tokens == 0


def _sched(blocks=8, bs=16, seqs=3):
    cfg = Config("x", hf_config=TafopelConfig(th.config_a()), max_num_seqs=seqs, max_num_batched_tokens=256, max_model_len=128,
                 kvcache_block_size=bs, num_kvcache_blocks=blocks)
    cfg.num_state_slots, cfg.prefix_cache = seqs, False
    Sequence.block_size = bs
    return Scheduler(cfg)


def test_plan_step_mixes_portions_and_single_tokens():
    s = _sched()
    first = list(range(1, 18))
    a, b = Sequence(first), Sequence([7])
    batch, varlen = s.plan_step([(a, first), (b, [7])])
    assert varlen and [q.num_scheduled_tokens for q in batch] == [17, 1] and len(a.block_table) == 2 and b.state_slot == 1
    s.postprocess_replay(batch)
    batch, varlen = s.plan_step([(a, [6]), (b, [8, 9])])           # one decodes while the other brings a portion
    assert varlen and a.num_tokens == 18 and b.token_ids == [7, 8, 9]
    s.postprocess_replay(batch)
    batch, varlen = s.plan_step([(b, [1]), (a, [2])])
    assert not varlen and all(not q.is_prefill for q in batch)     # one token each on top of cached ones: a decode step
    s.postprocess_replay(batch)
    pages = list(a.block_table)
    s.retire(a)
    c = Sequence([3] * 100)
    batch, _ = s.plan_step([(c, [3] * 100)])
    assert c.state_slot == 0 and set(pages) <= set(c.block_table)  # a's slot and pages are used again
    with pytest.raises(RuntimeError):
        s.plan_step([(Sequence([1] * 20), [1] * 20)])             # the pool is dictated, not grown


def test_engine_scheduler_gives_and_takes_slots():
    """The generation path: admission takes a slot with the blocks, preemption and completion return it."""
    s = _sched(blocks=4, bs=16, seqs=2)
    a, b = Sequence([1] * 32), Sequence([2] * 32)
    s.add(a), s.add(b)
    batch, is_prefill = s.schedule()
    assert is_prefill and batch == [a, b] and (a.state_slot, b.state_slot) == (0, 1)
    s.postprocess(batch, [5, 6], True)
    batch, is_prefill = s.schedule()               # both need a third page and there is none: b goes back to waiting, then a too
    assert not is_prefill or batch
    assert b.state_slot == -1 and not b.block_table                 # preempted: its pages and its slot are returned
    for q in (a, b):
        if q.block_table:
            s.retire(q)
    assert sorted(s.block_manager.free_state_slots) == [0, 1] and len(s.block_manager.free_block_ids) == 4


def test_plain_implementation_is_causal_and_its_scan_matches_a_closed_form():
    cfg, W = th.config_a(), th.random_weights(th.config_a(), 3)
    toks = th.tokens(12, cfg["vocab"], 0)
    full = ref.forward(cfg, W, toks)
    assert torch.allclose(ref.forward(cfg, W, toks[:7]), full[:7], atol=1e-9)
    # one channel, one state, constant input: S_t = sum_k decay^k * dt * u * B
    m = {"inner": 1, "state": 1, "dt_rank": 1, "conv": 1}
    one = lambda v: torch.tensor(v, dtype=torch.float64)
    Wm = {"p.in": one([[1.0], [0.0]]), "p.conv": one([[1.0]]), "p.conv.b": one([0.0]), "p.x": one([[1.0], [1.0], [1.0]]),
          "p.dt": one([[0.0]]), "p.dt.b": one([0.5]), "p.A_log": one([[0.0]]), "p.D": one([0.0]), "p.o": one([[1.0]])}
    h = torch.ones(5, 1, dtype=torch.float64)
    u = torch.nn.functional.silu(one(1.0))
    dt = torch.nn.functional.softplus(one(0.5))
    S, want = 0.0, []
    for _ in range(5):
        S = torch.exp(-dt) * S + dt * u * u
        want.append(S * u * 0.5 * 0.0 + S * u * 0.0 + (S * u) * (0.0 * torch.sigmoid(one(0.0))))
    got = ref.mamba1(h, Wm, "p.", m)
    assert torch.allclose(got.view(-1), torch.zeros(5, dtype=torch.float64))      # z = 0 gates everything off
    Wm["p.in"] = one([[1.0], [1.0]])
    got = ref.mamba1(h, Wm, "p.", m).view(-1)
    S, want = 0.0, []
    for _ in range(5):
        S = torch.exp(-dt) * S + dt * u * u
        want.append(S * u * torch.nn.functional.silu(one(1.0)))
    assert torch.allclose(got, torch.stack(want), atol=1e-12)


def test_mixer_library_header_and_binding_agree():
    """Every entry point include/b200_mixers.h declares is typed in the ctypes table (and exported, when the library is built)."""
    import ctypes
    import re
    from nanovllm import _native as nat
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    text = re.sub(r"/\*.*?\*/", "", open(os.path.join(root, "include", "b200_mixers.h")).read(), flags=re.S)
    names = sorted(set(re.findall(r"\b(b200m_[a-z0-9_]+)\s*\(", text)))
    assert len(names) >= 14 and set(names) == set(nat.MIX_SIGNATURES)
    for n in names:                      # argument counts of the prototypes match the table
        proto = re.search(r"\b%s\s*\(([^;]*?)\)\s*;" % n, text, flags=re.S).group(1).strip()
        argc = 0 if proto in ("", "void") else proto.count(",") + 1
        assert argc == len(nat.MIX_SIGNATURES[n][1]), n
    if nat.mix_lib_path().exists():
        lib = ctypes.CDLL(str(nat.mix_lib_path()))
        for n in names:
            assert hasattr(lib, n), n
