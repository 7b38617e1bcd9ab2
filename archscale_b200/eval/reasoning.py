"""Reasoning benchmarks (AIME 2024 / 2025, MATH-500, GPQA main / diamond): prompts, answer extraction, pass@1.

The reference defines these as custom LightEval tasks (`eval_reason/eval_reason.py:75-241`) and leaves generation,
extraction and scoring to LightEval + vLLM (`eval_reason/eval_reason.sh`).  This module carries the task definitions
(same prompts, datasets, sample counts and generation budget) and adds what is needed to run them without either
package: a ``\\boxed{}`` extractor with math normalisation, the unbiased pass@1 estimate over ``n`` samples, and a runner
over local JSONL copies of the datasets that uses :class:`archscale_b200.eval.common.ModelWrapper` for generation.
:func:`lighteval_tasks` returns ``LightevalTaskConfig`` objects for users who have LightEval installed.
"""
from __future__ import annotations

import json
import math
import random
import re
from dataclasses import dataclass
from fractions import Fraction
from typing import Callable, Dict, Iterable, List, Optional, Sequence

MATH_QUERY_TEMPLATE = "Please reason step by step, and put your final answer within \\boxed{{}}. {Question}"
GPQA_QUERY_TEMPLATE = ("Please reason step by step, and put your final choice of one letter from A/B/C/D within \\boxed{{}}. "
                       "{Question}\n\nA) {A}\nB) {B}\nC) {C}\nD) {D}")


@dataclass
class Doc:
    task_name: str
    query: str
    choices: List[str]
    gold_index: int

    @property
    def gold(self) -> str:
        return self.choices[self.gold_index]


def math_prompt(line: Dict, task_name: str = "math_500") -> Doc:
    """MATH-500: the gold answer is the boxed expression of the reference solution."""
    return Doc(task_name, MATH_QUERY_TEMPLATE.format(Question=line["problem"]), [line["solution"]], 0)


def aime_prompt(line: Dict, task_name: str = "aime24") -> Doc:
    return Doc(task_name, MATH_QUERY_TEMPLATE.format(Question=line["problem"]), [str(line["answer"])], 0)


def gpqa_prompt(line: Dict, task_name: str = "gpqa_diamond", rng: Optional[random.Random] = None) -> Doc:
    """The correct answer is inserted at a random position among the three distractors."""
    rng = rng or random
    gold = rng.randint(0, 3)
    choices = [line["Incorrect Answer 1"], line["Incorrect Answer 2"], line["Incorrect Answer 3"]]
    choices.insert(gold, line["Correct Answer"])
    query = GPQA_QUERY_TEMPLATE.format(A=choices[0], B=choices[1], C=choices[2], D=choices[3], Question=line["Question"])
    return Doc(task_name, query, ["A", "B", "C", "D"], gold)


@dataclass
class ReasoningTask:
    name: str
    prompt_function: Callable[..., Doc]
    hf_repo: str
    hf_subset: str
    split: str
    n_samples: int               # samples per problem for pass@1
    kind: str                    # "math" (expression match) | "choice" (letter match)
    generation_size: int = 32768


TASKS: Dict[str, ReasoningTask] = {t.name: t for t in (
    ReasoningTask("aime24", aime_prompt, "HuggingFaceH4/aime_2024", "default", "train", 64, "math"),
    ReasoningTask("aime25", aime_prompt, "yentinglin/aime_2025", "default", "train", 64, "math"),
    ReasoningTask("math_500", math_prompt, "HuggingFaceH4/MATH-500", "default", "test", 8, "math"),
    ReasoningTask("gpqa", gpqa_prompt, "Idavidrein/gpqa", "gpqa_main", "train", 8, "choice"),
    ReasoningTask("gpqa_diamond", gpqa_prompt, "Idavidrein/gpqa", "gpqa_diamond", "train", 8, "choice"),
)}


# ------------------------------------------------------------------ answer extraction
def last_boxed(text: str) -> Optional[str]:
    """Content of the last ``\\boxed{...}`` (or ``\\fbox{...}``) with balanced braces; None if there is none."""
    best = None
    for m in re.finditer(r"\\(?:boxed|fbox)\s*\{", text):
        depth, i = 1, m.end()
        while i < len(text) and depth:
            depth += {"{": 1, "}": -1}.get(text[i], 0)
            i += 1
        if depth == 0:
            best = text[m.end():i - 1]
    return best


_STRIP = (("\\left", ""), ("\\right", ""), ("\\!", ""), ("\\,", ""), ("\;", ""), ("\\ ", ""), ("\\$", ""), ("$", ""),
          ("\\%", ""), ("%", ""), ("^\\circ", ""), ("^{\\circ}", ""), ("dfrac", "frac"), ("tfrac", "frac"), ("\\dots", ""))


def normalize_math(ans: str) -> str:
    s = ans.strip()
    s = re.sub(r"\\text\{([^}]*)\}", r"\1", s)
    s = re.sub(r"\\mbox\{([^}]*)\}", r"\1", s)
    for a, b in _STRIP:
        s = s.replace(a, b)
    s = re.sub(r"\\frac\s*(\d)\s*(\d)", r"\\frac{\1}{\2}", s)            # \frac12 → \frac{1}{2}
    s = re.sub(r"^[a-zA-Z]\s*=\s*", "", s)                                # "x = 5" → "5"
    s = s.replace(" ", "").rstrip(".")
    if re.fullmatch(r"-?\d{1,3}(,\d{3})+(\.\d+)?", s):
        s = s.replace(",", "")
    return s


def _as_number(s: str) -> Optional[Fraction]:
    m = re.fullmatch(r"(-?)\\frac\{(-?\d+)\}\{(-?\d+)\}", s)
    try:
        if m:
            return Fraction(int(m.group(2)), int(m.group(3))) * (-1 if m.group(1) else 1)
        if re.fullmatch(r"-?\d+/\d+", s):
            a, b = s.split("/")
            return Fraction(int(a), int(b))
        if re.fullmatch(r"-?\d+(\.\d+)?", s):
            return Fraction(s)
    except (ValueError, ZeroDivisionError):
        return None
    return None


def math_equal(pred: Optional[str], gold: str, precision: int = 5) -> bool:
    """Normalised string match, or numeric equality to ``precision`` decimals when both sides parse as numbers."""
    if pred is None:
        return False
    g = last_boxed(gold)
    a, b = normalize_math(pred), normalize_math(g if g is not None else gold)
    if a == b:
        return True
    x, y = _as_number(a), _as_number(b)
    return x is not None and y is not None and round(float(x), precision) == round(float(y), precision)


def extract_choice(text: str) -> Optional[str]:
    b = last_boxed(text)
    if b is not None:
        m = re.search(r"[A-D]", b.upper())
        if m:
            return m.group(0)
    m = re.findall(r"(?i)Answer[ \t]*:[ \t]*\(?([A-D])\)?", text)
    return m[-1].upper() if m else None


def is_correct(task: ReasoningTask, doc: Doc, completion: str) -> bool:
    if task.kind == "choice":
        return extract_choice(completion) == doc.gold
    return math_equal(last_boxed(completion), doc.gold)


def pass_at_k(n: int, c: int, k: int = 1) -> float:
    """Unbiased estimate of pass@k from ``c`` correct of ``n`` samples: 1 − C(n−c, k) / C(n, k)."""
    if n - c < k:
        return 1.0
    return 1.0 - math.prod(1.0 - k / i for i in range(n - c + 1, n + 1))


# ------------------------------------------------------------------ runner
def load_jsonl(path: str) -> List[Dict]:
    with open(path) as f:
        return [json.loads(l) for l in f if l.strip()]


def evaluate(task_name: str, lines: Iterable[Dict], generate: Callable[[str, int], Sequence[str]],
             n_samples: Optional[int] = None, seed: int = 0) -> Dict[str, float]:
    """``generate(prompt, n)`` returns ``n`` sampled completions.  Returns pass@1 averaged over the problems."""
    task = TASKS[task_name]
    n = n_samples or task.n_samples
    rng = random.Random(seed)
    scores = []
    for line in lines:
        doc = task.prompt_function(line, task.name, rng) if task.kind == "choice" else task.prompt_function(line, task.name)
        outs = generate(doc.query, n)
        c = sum(is_correct(task, doc, o) for o in outs)
        scores.append(pass_at_k(len(outs), c, 1))
    return {"task": task_name, "n_problems": len(scores), "n_samples": n,
            f"pass@1:{n}_samples": sum(scores) / max(len(scores), 1)}


def model_generator(wrapper, tokenizer, max_new_tokens: int = 32768, temperature: float = 0.6) -> Callable[[str, int], List[str]]:
    """Sampling generator on :class:`archscale_b200.eval.common.ModelWrapper` (n completions as one batch)."""
    import torch

    def gen(prompt: str, n: int) -> List[str]:
        ids = tokenizer.encode(prompt)
        ids = ids if isinstance(ids, torch.Tensor) else torch.tensor(ids)
        x = ids.to(wrapper.device).long().unsqueeze(0).repeat(n, 1)
        room = max(1, min(max_new_tokens, wrapper.config.block_size - x.shape[1]))
        out = wrapper.generate(x, max_gen_toks=room, do_sample=True, temperature=temperature,
                               eos_token_id=getattr(tokenizer, "eos_id", None))
        return [tokenizer.decode(s[x.shape[1]:].cpu()) for s in out.sequences]
    return gen


def lighteval_tasks():
    """The same tasks as ``LightevalTaskConfig`` objects (needs the ``lighteval`` package)."""
    from lighteval.metrics.metrics import Metrics
    from lighteval.tasks.lighteval_task import LightevalTaskConfig
    from lighteval.tasks.requests import Doc as LDoc
    metric = {64: "math_pass_at_1_64n", 8: "math_pass_at_1_8n"}
    table = []
    for t in TASKS.values():
        def fn(line, task_name=None, _t=t):
            d = _t.prompt_function(line, task_name or _t.name)
            return LDoc(task_name=task_name, query=d.query, choices=d.choices, gold_index=d.gold_index)
        m = getattr(Metrics, "gpqa_instruct_pass_at_1_8n" if t.kind == "choice" else metric[t.n_samples])
        table.append(LightevalTaskConfig(name=t.name, suite=["custom"], prompt_function=fn, hf_repo=t.hf_repo, hf_subset=t.hf_subset,
                                         hf_avail_splits=[t.split], evaluation_splits=[t.split], few_shots_split=None,
                                         few_shots_select=None, generation_size=t.generation_size, metric=[m], version=1))
    return table


def main(argv: Optional[List[str]] = None) -> None:
    import argparse
    ap = argparse.ArgumentParser(description="pass@1 on a reasoning benchmark from a local JSONL copy of its dataset")
    ap.add_argument("--task", required=True, choices=sorted(TASKS))
    ap.add_argument("--data", required=True, help="JSONL file with the dataset's columns")
    ap.add_argument("--checkpoint", required=True)
    ap.add_argument("--config", required=True, help="model name in the registry")
    ap.add_argument("--tokenizer", required=True)
    ap.add_argument("--n_samples", type=int, default=None)
    ap.add_argument("--max_new_tokens", type=int, default=32768)
    ap.add_argument("--temperature", type=float, default=0.6)
    a = ap.parse_args(argv)
    from archscale_b200.data.tokenizer import Tokenizer
    from archscale_b200.eval.common import load_model
    wrapper = load_model(a.checkpoint, a.config)
    tok = Tokenizer(a.tokenizer)
    res = evaluate(a.task, load_jsonl(a.data), model_generator(wrapper, tok, a.max_new_tokens, a.temperature), a.n_samples)
    print(json.dumps(res))


if __name__ == "__main__":
    main()
