"""Table of multiple-choice evaluation tasks and the log-likelihood scoring they share (capability parity: reference
src/nanotron/eval/evaluation_tasks.py, which declares the same task families as ``lighteval`` task configs).

The reference only *declares* tasks and leaves prompting, batching and scoring to the ``lighteval`` package.  That package is an
optional dependency here: the table below is self-contained (``EvalTask`` carries the dataset coordinates, a line adapter and a
prompt formulation), ``nanotron_b200.eval.harness`` scores it with this framework's own models, and ``to_lighteval`` converts
the table when ``lighteval`` is importable.

Formulations (what the model is asked to continue):
  * ``MCF``    multiple-choice: the options are listed with letters, the continuations are the letters;
  * ``CF``     cloze: no options in the prompt, the continuations are the option texts;
  * ``HYBRID`` options listed, continuations are the option texts.
Metrics: accuracy of the arg-max continuation under three normalisations of its summed log-probability -- per token, per
character, and PMI (minus the log-probability of the same continuation after a context-free prompt).
"""
from __future__ import annotations

import dataclasses
import enum
import math
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

LETTER_INDICES = ["A", "B", "C", "D", "E", "F", "G", "H", "I", "J", "K", "L", "M", "N", "O", "P", "Q", "R", "S", "T", "U", "V", "W", "X", "Y", "Z"]


class Formulation(enum.Enum):
    MCF = "mcf"
    CF = "cf"
    HYBRID = "hybrid"


@dataclasses.dataclass(frozen=True)
class MCQDoc:
    """One question after its task's adapter: free-text context (may be empty), question, options, index of the right one."""

    question: str
    choices: Tuple[str, ...]
    gold_idx: int
    context: str = ""
    continuation_prefix: str = ""  # text of the question repeated in front of every continuation (cloze-by-sentence tasks)


@dataclasses.dataclass(frozen=True)
class EvalTask:
    name: str
    hf_repo: str
    hf_subset: Optional[str]
    adapter: Callable[[Dict[str, Any]], MCQDoc]
    formulation: Formulation
    evaluation_splits: Tuple[str, ...] = ("test",)
    few_shots_split: Optional[str] = None
    hf_revision: Optional[str] = None
    suite: Tuple[str, ...] = ("custom",)
    metrics: Tuple[str, ...] = ("acc_token", "acc_char", "acc_pmi")


@dataclasses.dataclass(frozen=True)
class Request:
    """``continuations[i]`` scored after ``prompt``; ``unconditioned_prompt`` is the context-free prompt of the PMI normalisation."""

    prompt: str
    continuations: Tuple[str, ...]
    gold_idx: int
    unconditioned_prompt: str = "Answer:"


# ---------------------------------------------------------------------------- prompts
def build_request(task: EvalTask, line: Dict[str, Any], few_shots: Sequence[Dict[str, Any]] = ()) -> Request:
    """Prompt and continuations of one dataset line (``few_shots``: solved lines of the few-shot split placed in front)."""
    doc = task.adapter(line)
    shots = "".join(_render(task.formulation, task.adapter(s), with_answer=True) + "\n\n" for s in few_shots)
    prompt = shots + _render(task.formulation, doc, with_answer=False)
    if task.formulation is Formulation.MCF:
        conts = tuple(f" {LETTER_INDICES[i]}" for i in range(len(doc.choices)))
    else:
        conts = tuple(f" {doc.continuation_prefix}{c}".rstrip() if doc.continuation_prefix else f" {c}" for c in doc.choices)
    return Request(prompt=prompt, continuations=conts, gold_idx=doc.gold_idx)


def _render(formulation: Formulation, doc: MCQDoc, with_answer: bool) -> str:
    parts = []
    if doc.context:
        parts.append(doc.context.strip())
    if doc.question:
        parts.append(f"Question: {doc.question.strip()}")
    if formulation in (Formulation.MCF, Formulation.HYBRID):
        parts.extend(f" {LETTER_INDICES[i]}. {c.strip()}" for i, c in enumerate(doc.choices))
    parts.append("Answer:")
    text = "\n".join(parts)
    if with_answer:
        gold = LETTER_INDICES[doc.gold_idx] if formulation is Formulation.MCF else doc.choices[doc.gold_idx]
        text += f" {gold}"
    return text


# ---------------------------------------------------------------------------- scoring
def choice_scores(logprobs: Sequence[float], continuations: Sequence[str], num_tokens: Sequence[int], unconditioned_logprobs: Optional[Sequence[float]] = None) -> Dict[str, List[float]]:
    """Normalised scores of every continuation: summed log-probability per token, per character, and PMI."""
    out = {
        "acc_token": [lp / max(n, 1) for lp, n in zip(logprobs, num_tokens)],
        "acc_char": [lp / max(len(c.strip()), 1) for lp, c in zip(logprobs, continuations)],
    }
    if unconditioned_logprobs is not None:
        out["acc_pmi"] = [lp - u for lp, u in zip(logprobs, unconditioned_logprobs)]
    return out


def accuracy(scores: Dict[str, List[float]], gold_idx: int) -> Dict[str, float]:
    return {name: float(max(range(len(vals)), key=lambda i: (vals[i], -i)) == gold_idx) for name, vals in scores.items()}


def aggregate(per_doc: Sequence[Dict[str, float]]) -> Dict[str, float]:
    """Mean and standard error of every metric over the documents of a task."""
    out: Dict[str, float] = {}
    if not per_doc:
        return out
    for name in per_doc[0]:
        vals = [d[name] for d in per_doc if name in d]
        mean = sum(vals) / len(vals)
        var = sum((v - mean) ** 2 for v in vals) / max(len(vals) - 1, 1)
        out[name] = mean
        out[name + "_stderr"] = math.sqrt(var / len(vals))
    return out


# ---------------------------------------------------------------------------- adapters (dataset line -> MCQDoc)
def _letter_or_digit(key: str) -> int:
    key = str(key).strip()
    return int(key) - 1 if key.isdigit() else LETTER_INDICES.index(key)


def arc_adapter(line) -> MCQDoc:
    return MCQDoc(question=line["question"], choices=tuple(line["choices"]["text"]), gold_idx=_letter_or_digit(line["answerKey"]))


def hellaswag_adapter(line) -> MCQDoc:
    ctx = f"{line['ctx_a']} {line['ctx_b'].capitalize()}".strip()
    return MCQDoc(question="", context=f"{line['activity_label']}: {ctx}", choices=tuple(line["endings"]), gold_idx=int(line["label"]))


def commonsenseqa_adapter(line) -> MCQDoc:
    return MCQDoc(question=line["question"], choices=tuple(line["choices"]["text"]), gold_idx=list(line["choices"]["label"]).index(str(line["answerKey"]).strip()))


def openbookqa_adapter(line) -> MCQDoc:
    return MCQDoc(question=line["question_stem"], choices=tuple(line["choices"]["text"]), gold_idx=LETTER_INDICES.index(str(line["answerKey"]).strip()))


def winogrande_adapter(line) -> MCQDoc:
    """The blank splits the sentence: the part before it (with either option filled in) is the context-dependent continuation
    prefix, the part after it is what both candidates are scored on."""
    before, _, after = line["sentence"].partition("_")
    return MCQDoc(question="", context="", choices=tuple(f"{before}{o}{after}".strip() for o in (line["option1"], line["option2"])), gold_idx=int(line["answer"]) - 1)


def piqa_adapter(line) -> MCQDoc:
    return MCQDoc(question=line["goal"], choices=(line["sol1"], line["sol2"]), gold_idx=int(line["label"]))


def mmlu_adapter(line) -> MCQDoc:
    return MCQDoc(question=line["question"], choices=tuple(line["choices"]), gold_idx=int(line["answer"]))


def mmlu_pro_adapter(line) -> MCQDoc:
    return MCQDoc(question=line["question"], choices=tuple(line["options"]), gold_idx=int(line["answer_index"]))


MMLU_SUBSETS = [
    "abstract_algebra", "anatomy", "astronomy", "business_ethics", "clinical_knowledge", "college_biology", "college_chemistry", "college_computer_science",
    "college_mathematics", "college_medicine", "college_physics", "computer_security", "conceptual_physics", "econometrics", "electrical_engineering",
    "elementary_mathematics", "formal_logic", "global_facts", "high_school_biology", "high_school_chemistry", "high_school_computer_science",
    "high_school_european_history", "high_school_geography", "high_school_government_and_politics", "high_school_macroeconomics", "high_school_mathematics",
    "high_school_microeconomics", "high_school_physics", "high_school_psychology", "high_school_statistics", "high_school_us_history", "high_school_world_history",
    "human_aging", "human_sexuality", "international_law", "jurisprudence", "logical_fallacies", "machine_learning", "management", "marketing", "medical_genetics",
    "miscellaneous", "moral_disputes", "moral_scenarios", "nutrition", "philosophy", "prehistory", "professional_accounting", "professional_law",
    "professional_medicine", "professional_psychology", "public_relations", "security_studies", "sociology", "us_foreign_policy", "virology", "world_religions",
]


def _family(name: str, repo: str, subset: Optional[str], adapter, splits=("test",), few=None, formulations=tuple(Formulation), sep="_") -> List[EvalTask]:
    return [
        EvalTask(name=name.format(f=f.value), hf_repo=repo, hf_subset=subset, adapter=adapter, formulation=f, evaluation_splits=tuple(splits), few_shots_split=few,
                 metrics=("acc_token", "acc_char", "acc_pmi") if f is not Formulation.MCF else ("acc_token",))
        for f in formulations
    ]


TASKS_TABLE: List[EvalTask] = []
for _subset in ("Easy", "Challenge"):
    TASKS_TABLE += _family("arc_{f}:" + _subset.lower(), "allenai/ai2_arc", f"ARC-{_subset}", arc_adapter, few="train")
TASKS_TABLE += _family("hellaswag_{f}", "Rowan/hellaswag", "default", hellaswag_adapter, splits=("validation",), few="train")
TASKS_TABLE += _family("commonsenseqa_{f}", "tau/commonsense_qa", "default", commonsenseqa_adapter, splits=("validation",), few="train")
TASKS_TABLE += _family("openbookqa_{f}", "allenai/openbookqa", "main", openbookqa_adapter, few="train")
TASKS_TABLE += _family("winogrande_{f}", "allenai/winogrande", "winogrande_xl", winogrande_adapter, splits=("validation",), few="train", formulations=(Formulation.CF,))
TASKS_TABLE += _family("piqa_{f}", "ybisk/piqa", "plain_text", piqa_adapter, splits=("validation",), few="train")
for _subset in MMLU_SUBSETS:
    TASKS_TABLE += _family("mmlu_{f}:" + _subset, "cais/mmlu", _subset, mmlu_adapter, few="dev")
TASKS_TABLE += _family("mmlu_pro_{f}", "TIGER-Lab/MMLU-Pro", "default", mmlu_pro_adapter, few="validation")
TASKS_BY_NAME: Dict[str, EvalTask] = {t.name: t for t in TASKS_TABLE}


def get_tasks(spec: str) -> List[EvalTask]:
    """Tasks named by a comma-separated list; a trailing ``*`` matches a prefix (``mmlu_cf:*``), ``all`` means the whole table."""
    if spec.strip() == "all":
        return list(TASKS_TABLE)
    out: List[EvalTask] = []
    for item in (s.strip() for s in spec.split(",") if s.strip()):
        if item.endswith("*"):
            hits = [t for t in TASKS_TABLE if t.name.startswith(item[:-1])]
            assert hits, f"no task matches {item!r}"
            out += hits
        else:
            assert item in TASKS_BY_NAME, f"unknown task {item!r}"
            out.append(TASKS_BY_NAME[item])
    return out


def to_lighteval(tasks: Optional[Sequence[EvalTask]] = None):
    """The same tasks as ``lighteval`` task configs (needs the ``lighteval`` package)."""
    try:
        from lighteval.metrics.dynamic_metrics import loglikelihood_acc_metric
        from lighteval.metrics.normalizations import LogProbCharNorm, LogProbPMINorm, LogProbTokenNorm
        from lighteval.tasks.lighteval_task import LightevalTaskConfig
        from lighteval.tasks.requests import Doc
    except ImportError as e:
        raise ImportError("to_lighteval needs the optional `lighteval` package") from e
    norms = {"acc_token": LogProbTokenNorm, "acc_char": LogProbCharNorm, "acc_pmi": LogProbPMINorm}
    out = []
    for t in tasks if tasks is not None else TASKS_TABLE:
        def prompt_fn(line, task_name=None, t=t):
            r = build_request(t, line)
            return Doc(task_name=task_name, query=r.prompt, choices=list(r.continuations), gold_index=r.gold_idx, unconditioned_query=r.unconditioned_prompt)

        out.append(LightevalTaskConfig(
            name=t.name, prompt_function=prompt_fn, suite=t.suite, hf_repo=t.hf_repo, hf_subset=t.hf_subset, hf_revision=t.hf_revision, trust_dataset=True,
            evaluation_splits=t.evaluation_splits, few_shots_split=t.few_shots_split, metric=[loglikelihood_acc_metric(normalization=norms[m]()) for m in t.metrics],
        ))
    return out


if __name__ == "__main__":
    print(*[t.name for t in TASKS_TABLE], sep="\n")
    print(len(TASKS_TABLE))
