"""Host side of serving, no GPU: checkpoint files, the model registry and Lilovik's configuration, the page /
state-slot manager, the scheduler's mixed batches, and the engine loop over a stand-in executor."""
import json

import pytest
import torch

from atoma_infer_b200 import checkpoint, lilovik, models
from atoma_infer_b200.cache import CacheManager, FreeList, OutOfPages, OutOfStateSlots
from atoma_infer_b200.engine import Engine
from atoma_infer_b200.hybrid import StepOutput, slopes_power_of_two
from atoma_infer_b200.ops import AtomaError
from atoma_infer_b200.scheduler import SamplingParams, Scheduler, Sequence

import lilovik_oracle as lo


def test_safetensors_round_trip(tmp_path):
    g = torch.Generator().manual_seed(0)
    t = {"a": torch.randn(3, 5, generator=g).to(torch.bfloat16), "b.c": torch.arange(7, dtype=torch.int32),
         "d": torch.randn(2, 2, 2, generator=g)}
    checkpoint.write_safetensors(tmp_path / "model.safetensors", t, metadata={"k": "v"})
    f = checkpoint.SafetensorsFile(tmp_path / "model.safetensors")
    assert set(f.keys()) == set(t) and f.metadata == {"k": "v"} and f.shape("a") == (3, 5)
    for k in t:
        assert f[k].dtype == t[k].dtype and torch.equal(f[k], t[k])
    assert set(checkpoint.open_checkpoint(tmp_path)) == set(t)


def test_safetensors_rejects_bad_offsets(tmp_path):
    import struct
    h = json.dumps({"x": {"dtype": "F32", "shape": [4], "data_offsets": [0, 12]}}).encode()
    (tmp_path / "m.safetensors").write_bytes(struct.pack("<Q", len(h)) + h + b"\0" * 16)
    with pytest.raises(ValueError):
        checkpoint.SafetensorsFile(tmp_path / "m.safetensors")


def test_registry_resolves_by_architecture():
    assert models.resolve({"architecture": "Lilovik"}).name == "Lilovik"
    assert models.resolve({"architectures": ["LlamaForCausalLM"]}).name == "LlamaForCausalLM"
    with pytest.raises(AtomaError):
        models.resolve({"architecture": "nope"})
    with pytest.raises(AtomaError):
        models.resolve({})


def test_lilovik_spec_and_weight_layout():
    g = torch.Generator().manual_seed(1)
    cfg = lo.random_config(g, layers=("mingru", "attention"), heads=6, kv_heads=3, dim=8, vdim=16, state=24, width=40, ff=56,
                           mlp_on_mingru=True)
    spec = lilovik.spec_from_config(cfg)
    assert spec.has_state and spec.norm_offset == 1.0 and [l.mixer for l in spec.layers] == ["mingru", "attention"]
    a = spec.layers[1].attention
    assert (a.heads, a.kv_heads, a.dim, a.vdim) == (6, 3, 8, 16)
    assert list(a.slopes) == pytest.approx([2.0 ** (-8.0 * (h + 1) / 6) for h in range(6)])
    assert slopes_power_of_two(1) == [2.0 ** -8]
    assert spec.layers[0].mlp.ff == 56 and spec.layers[0].mlp.act == "relu"
    assert spec.cache_bytes_per_token(torch.bfloat16) == 3 * (8 + 16) * 2
    w = lo.random_weights(cfg, g, dtype=torch.float32)
    lay = lilovik.weights_from_checkpoint(spec, w)
    assert lay["layers"][1]["w_qkv"].shape == (6 * 8 + 3 * 8 + 3 * 16, 40)
    assert torch.equal(lay["layers"][1]["w_qkv"][48:72], w["l1.mix.k"])
    assert lay["layers"][0]["w_zxg"].shape == (72, 40) and torch.count_nonzero(lay["layers"][0]["b_zxg"][48:]) == 0
    assert lay["layers"][0]["w_gate_up"].shape == (112, 40)
    bad = dict(w)
    bad["l1.mix.q"] = bad["l1.mix.q"][:-1]
    with pytest.raises(AtomaError):
        lilovik.weights_from_checkpoint(spec, bad)
    del bad["l1.mix.q"]
    with pytest.raises(AtomaError):
        lilovik.weights_from_checkpoint(spec, bad)
    cfg["layers"][0]["type"] = "lstm"
    with pytest.raises(AtomaError):
        lilovik.spec_from_config(cfg)


def test_free_list_is_lifo_and_checks_handles():
    f = FreeList(3)
    a, b = f.take(), f.take()
    assert (a, b) == (0, 1)
    f.give_back(a)
    assert f.take() == a                       # the most recently freed handle is the next one out
    with pytest.raises(ValueError):
        f.give_back(2)


def test_cache_manager_pages_and_slots_are_reused():
    cm = CacheManager(num_blocks=6, block_size=4, num_state_slots=2)
    cm.admit("a")
    cm.grow("a", 9)
    assert len(cm.get("a").block_table) == 3 and cm.get("a").state_slot == 0
    cm.admit("b")
    cm.grow("b", 4)
    assert not cm.can_admit(1)                 # both slots taken
    with pytest.raises(OutOfStateSlots):
        cm.admit("c")
    assert cm.blocks_needed("b", 13) == 3 and not cm.can_grow("b", 13)
    with pytest.raises(OutOfPages):
        cm.grow("b", 13)
    assert len(cm.get("b").block_table) == 1   # all-or-nothing
    pages_a, slot_a = list(cm.get("a").block_table), cm.get("a").state_slot
    cm.free("a")
    cm.admit("c")
    cm.grow("c", 12)
    assert cm.get("c").state_slot == slot_a and set(cm.get("c").block_table) == set(pages_a)
    assert cm.live == 2
    no_state = CacheManager(4, 4, 0)
    no_state.admit("x")
    assert no_state.get("x").state_slot is None and no_state.can_admit(16) and not no_state.can_admit(17)


def _seq(i, n, new=4):
    return Sequence(f"s{i}", list(range(n)), n, SamplingParams(max_new_tokens=new))


def test_scheduler_chunks_prompts_and_mixes_them_with_decodes():
    cm = CacheManager(64, 4, 4)
    sch = Scheduler(cm, max_num_batched_tokens=10, max_num_seqs=4)
    a, b = _seq(0, 7), _seq(1, 25)
    sch.add(a)
    sch.add(b)
    p = sch.plan()
    assert [(c.seq.seq_id, c.start, c.count, c.want) for c in p.chunks] == [("s0", 0, 7, (6,)), ("s1", 0, 3, ())]
    sch.commit(p)
    a.tokens.append(99)                        # the engine appends the sampled token
    p = sch.plan()
    assert [(c.seq.seq_id, c.start, c.count, c.want) for c in p.chunks] == [("s0", 7, 1, (0,)), ("s1", 3, 9, ())]
    assert p.chunks[0].is_decode and not p.chunks[1].is_decode
    assert len(p.chunks[1].block_table) == 3 and p.chunks[1].state_slot == 1
    sch.commit(p)
    sch.finish(a)
    assert "s0" not in cm and sch.running == [b]


def test_scheduler_admits_only_while_slots_and_pages_last_and_preempts():
    cm = CacheManager(num_blocks=4, block_size=4, num_state_slots=2)
    sch = Scheduler(cm, max_num_batched_tokens=64, max_num_seqs=8)
    s = [_seq(i, 6) for i in range(3)]
    for x in s:
        sch.add(x)
    p = sch.plan()
    assert [c.seq.seq_id for c in p.chunks] == ["s0", "s1"] and list(sch.waiting) == [s[2]]   # two slots, four pages
    sch.commit(p)
    for x in s[:2]:
        x.tokens += [1, 2, 3]                  # both now need a third page; only the older one can have it
    p = sch.plan()
    assert p.preempted == ["s1"] and [c.seq.seq_id for c in p.chunks] == ["s0"]
    assert s[1].num_computed == 0 and sch.waiting[0] is s[1] and "s1" not in cm


def test_forced_plans_use_the_same_allocations():
    cm = CacheManager(8, 4, 2)
    sch = Scheduler(cm, 64, 4)
    a = Sequence("a", [1, 2, 3, 4, 5], 5)
    p = sch.plan_forced([(a, 2, [1])])
    assert p.chunks[0].start == 0 and p.chunks[0].want == (1,) and len(p.chunks[0].block_table) == 1
    sch.commit(p)
    p = sch.plan_forced([(a, 3, [])])
    assert p.chunks[0].start == 2 and len(p.chunks[0].block_table) == 2
    sch.commit(p)
    with pytest.raises(ValueError):
        sch.plan_forced([(a, 1, [])])          # nothing pending


class _CountingExecutor:
    """next token = (last token of the chunk + position) % 50; records the batches it was given."""

    def __init__(self):
        self.batches = []

    def execute(self, plan, **kw):
        self.batches.append([(c.seq.seq_id, c.start, c.count) for c in plan.chunks])
        rows, toks = [], []
        for c in plan.chunks:
            for w in c.want:
                rows.append((c.seq.seq_id, w))
                toks.append((c.seq.tokens[c.start + w] + c.start + w) % 50)
        return StepOutput(None, torch.tensor(toks, dtype=torch.int32) if toks else None, rows)


def test_engine_generates_through_the_scheduler_with_few_slots():
    ex = _CountingExecutor()
    eng = Engine(ex, CacheManager(num_blocks=12, block_size=4, num_state_slots=2), max_num_batched_tokens=8, max_num_seqs=2)
    prompts = [[3, 4, 5], [7] * 11, [9, 9]]
    got = eng.generate(prompts, max_new_tokens=3)

    def alone(p):
        t = list(p)
        for _ in range(3):
            t.append((t[-1] + len(t) - 1) % 50)
        return t[len(p):]

    assert got == [alone(p) for p in prompts]
    assert eng.cache.live == 0 and eng.cache.blocks.num_free == 12 and eng.cache.state_slots.num_free == 2
    assert any(len(b) == 2 and {c for _, _, c in b} != {1} for b in ex.batches)   # a prompt portion beside a decoded token
    assert max(len(b) for b in ex.batches) <= 2


def test_engine_forced_steps_admit_extend_and_end():
    ex = _CountingExecutor()
    eng = Engine(ex, CacheManager(8, 4, 2))
    eng.step_forced([("a", [1, 2, 3], [2]), ("b", [5], [])])
    eng.step_forced([("a", [4], [0])], end=["a"])
    assert ex.batches == [[("a", 0, 3), ("b", 0, 1)], [("a", 3, 1)]]
    assert "a" not in eng.sequences and eng.cache.live == 1
    eng.step_forced([("c", [1] * 9, [])])
    assert eng.cache.get("c").state_slot == 0      # a's slot, used again
