"""Llama through the serving engine: the mixed-batch executor agrees with itself across schedules and with the
decode-step executor (llama.DecodeStep) that the decode benchmarks replay."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _engine(live=3, budget=64):
    from atoma_infer_b200.cache import CacheManager
    from atoma_infer_b200.engine import Engine
    from atoma_infer_b200.llama import LlamaConfig, LlamaShard
    from atoma_infer_b200.llama_engine import LlamaExecutor
    cfg = LlamaConfig(hidden_size=256, intermediate_size=512, vocab_size=320, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, max_position_embeddings=512)
    shard = LlamaShard.random_init(cfg, device=DEV, seed=9, gen_device="cpu")
    ex = LlamaExecutor(shard, num_blocks=40, block_size=16)
    return Engine(ex, CacheManager(40, 16, 0), max_num_batched_tokens=budget, max_num_seqs=live), shard


def nerr(a, b):
    a, b = a.double().cpu(), b.double().cpu()
    return float(((a - b) ** 2).mean().sqrt() / (b ** 2).mean().sqrt())


def test_portions_and_mixed_batches_equal_the_whole_prompt():
    g = torch.Generator().manual_seed(0)
    a = torch.randint(0, 320, (150,), generator=g).tolist()
    b = torch.randint(0, 320, (37,), generator=g).tolist()
    eng, _ = _engine()
    whole_a = eng.step_forced([("a", a, list(range(150)))], end=["a"]).logits.clone()
    whole_b = eng.step_forced([("b", b, list(range(37)))], end=["b"]).logits.clone()
    got_a, got_b = [], []
    out = eng.step_forced([("a", a[:100], list(range(100))), ("b", b[:36], list(range(36)))])
    got_a.append(out.logits[:100].clone())
    got_b.append(out.logits[100:].clone())
    out = eng.step_forced([("b", b[36:], [0]), ("a", a[100:102], [0, 1])], end=["b"])
    got_b.append(out.logits[:1].clone())
    got_a.append(out.logits[1:].clone())
    for t in a[102:]:
        got_a.append(eng.step_forced([("a", [t], [0])]).logits.clone())
    assert nerr(torch.cat(got_a), whole_a) < 2e-2 and nerr(torch.cat(got_b), whole_b) < 2e-2


def test_the_engine_path_agrees_with_the_decode_step_executor():
    from atoma_infer_b200.llama import DecodeStep
    g = torch.Generator().manual_seed(1)
    toks = torch.randint(0, 320, (70,), generator=g).tolist()
    eng, shard = _engine()
    eng.step_forced([("a", toks[:-1], [])])
    kv = [c.clone() for c in eng.executor.kv_caches]
    want = eng.step_forced([("a", toks[-1:], [0])]).logits.clone()
    bt = torch.tensor([list(eng.cache.get("a").block_table) + [0] * 3], dtype=torch.int32, device=DEV)
    n = len(toks)
    pos = torch.tensor([n - 1], dtype=torch.int64, device=DEV)
    slot = bt[0, (n - 1) // 16].long() * 16 + (n - 1) % 16
    step = DecodeStep(shard, kv, max_batch=1, want_logits_f32=True)
    step.bind(torch.tensor(toks[-1:], dtype=torch.int32, device=DEV), pos, slot.reshape(1), bt,
              torch.tensor([n], dtype=torch.int32, device=DEV))
    step.launch()
    torch.cuda.synchronize()
    assert nerr(step.logits_f32[:1], want) < 2e-2
    assert int(step.next_tokens[0]) == int(want.argmax())


def test_greedy_generation_through_the_scheduler():
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, 320, (n,), generator=g).tolist() for n in (90, 5, 33, 17)]
    eng, _ = _engine(live=2, budget=48)
    got = eng.generate(prompts, max_new_tokens=5)
    assert [len(x) for x in got] == [5] * 4 and eng.cache.live == 0
    eng2, _ = _engine(live=4, budget=512)
    assert eng2.generate(prompts, max_new_tokens=1) == [x[:1] for x in got]
