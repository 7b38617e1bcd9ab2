"""Evaluation helpers on CPU: path-convention config, generation, sliding-window loss, phonebook prompts."""
import math

import numpy as np
import torch

from archscale_b200.config import Config
from archscale_b200.eval import ModelWrapper, config_from_checkpoint_path
from archscale_b200.eval import phonebook, proofpile
from archscale_b200.models.gpt import GPT


def _tiny():
    cfg = Config.from_name("transformer_gqa4_d8", vocab_size=64, block_size=64, n_layer=2, n_embd=64, n_head=2,
                           n_query_groups=1, head_dim=32, intermediate_size=128)
    torch.manual_seed(0)
    m = GPT(cfg)
    with torch.no_grad():
        for p in m.parameters():
            p.normal_(0, 0.1) if p.dim() > 1 else p.fill_(1.0)
    m.compute_dtype = torch.float32
    return cfg, m.float().eval()


def test_config_from_checkpoint_path():
    c = config_from_checkpoint_path("out/scaling_mup_tie_rbase_sambay_d16_ctx32768_swa1024/iter-1-ckpt.pth", "sambay_d16")
    assert c.mup and c.tied_embed and c.rope_base == 640000 and c.local_window == 1024 and c.block_size == 32768
    assert c.scaling_factor == 32768 / (8192 if c.yoco_window else 4096)


def test_generate_greedy_matches_stepwise_argmax():
    cfg, m = _tiny()
    w = ModelWrapper(m)
    ids = torch.randint(0, 64, (2, 5))
    out = w.generate(ids, max_gen_toks=4, return_dict_in_generate=False)
    assert out.shape == (2, 9) and torch.equal(out[:, :5], ids)
    step = m(out[:, :8]).logits[:, -1].argmax(-1)
    assert torch.equal(step, out[:, 8])
    stopped = w.generate(ids, max_gen_toks=10, eos_token_id=int(out[0, 5]), return_dict_in_generate=False)
    assert stopped.shape[1] <= 15


def test_proofpile_windows_and_loss():
    cfg, m = _tiny()
    tokens = np.random.default_rng(0).integers(0, 64, size=200).astype(np.uint16)
    wins = list(proofpile.iter_windows(tokens, 32, 4, 16))
    assert sum(w.shape[0] for w in wins) == len(range(0, 200 - 32 + 1, 16)) and wins[0].shape[1] == 32
    res = proofpile.evaluate(m, tokens, seq_length=32, batch_size=4, sliding_window=16, device="cpu")
    ids = torch.from_numpy(tokens[:32].astype(np.int64))[None]
    ref = torch.nn.functional.cross_entropy(m(ids).logits[0, :-1, :64].float(), ids[0, 1:])
    assert abs(res["ppl"] - math.exp(res["loss"])) < 1e-6 and res["windows"] == 11
    one = proofpile.evaluate(m, tokens[:32], seq_length=32, batch_size=1, sliding_window=16, device="cpu")
    assert abs(one["loss"] - float(ref)) < 1e-3


def test_phonebook_prompts_are_reproducible_and_answerable():
    b1 = phonebook.make_batch(12, 4, seed=7)
    b2 = phonebook.make_batch(12, 4, seed=7)
    assert b1 == b2
    for prompt, label in zip(b1["input"], b1["label"]):
        q = prompt.rsplit("\n", 1)[-1]
        assert q.endswith(":") and f"{q} {label}" in prompt and len(label) == 10


def test_reasoning_tasks_extraction_and_pass_at_1():
    import random
    from archscale_b200.eval import reasoning as R
    assert set(R.TASKS) == {"aime24", "aime25", "math_500", "gpqa", "gpqa_diamond"}
    assert R.TASKS["aime24"].n_samples == 64 and R.TASKS["math_500"].n_samples == 8 and R.TASKS["aime24"].generation_size == 32768
    d = R.aime_prompt({"problem": "What is 1+1?", "answer": 2})
    assert d.query.startswith("Please reason step by step, and put your final answer within \\boxed{}.") and d.gold == "2"
    g = R.gpqa_prompt({"Question": "Q?", "Correct Answer": "yes", "Incorrect Answer 1": "a", "Incorrect Answer 2": "b",
                       "Incorrect Answer 3": "c"}, rng=random.Random(1))
    assert g.choices == ["A", "B", "C", "D"] and f"{g.gold}) yes" in g.query
    assert R.last_boxed("so \\boxed{1} then \\boxed{\\frac{3}{4}}.") == "\\frac{3}{4}"
    assert R.last_boxed("no box") is None
    assert R.math_equal("\\dfrac{3}{4}", "the answer is \\boxed{0.75}")
    assert R.math_equal("1,000", "1000") and R.math_equal("x=5", "5") and not R.math_equal("6", "5")
    assert R.extract_choice("... \\boxed{(C)}") == "C" and R.extract_choice("Answer: b") == "B"
    assert R.pass_at_k(8, 2, 1) == 0.25 and R.pass_at_k(4, 4, 1) == 1.0 and R.pass_at_k(4, 0, 1) == 0.0
    lines = [{"problem": "1+1", "answer": 2}, {"problem": "2+2", "answer": 4}]
    res = R.evaluate("aime24", lines, lambda prompt, n: ["\\boxed{2}"] * n, n_samples=4)
    assert res["n_problems"] == 2 and res["pass@1:4_samples"] == 0.5
