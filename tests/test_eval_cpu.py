"""Evaluation tasks and the in-tree log-likelihood harness: prompt formulations, normalised accuracies, and summed continuation
log-probabilities that match a direct computation from the full logits (single rank, and tp 2 x pp 2 on gloo)."""
import math

import torch

from helpers import make_config, run_distributed, tiny_llama_config
from nanotron_b200.eval import evaluation_tasks as et


def test_task_table_and_prompts():
    names = [t.name for t in et.TASKS_TABLE]
    assert len(names) == len(set(names))
    for must in ("arc_cf:easy", "arc_mcf:challenge", "hellaswag_hybrid", "commonsenseqa_cf", "openbookqa_mcf", "winogrande_cf", "piqa_cf", "mmlu_mcf:anatomy", "mmlu_pro_cf"):
        assert must in et.TASKS_BY_NAME, must
    assert len(et.get_tasks("mmlu_cf:*")) == len(et.MMLU_SUBSETS) == 57
    line = {"question": "Which is a mammal?", "choices": {"text": ["trout", "otter", "wasp"], "label": ["A", "B", "C"]}, "answerKey": "B"}
    mcf = et.build_request(et.TASKS_BY_NAME["arc_mcf:easy"], line)
    assert mcf.continuations == (" A", " B", " C") and mcf.gold_idx == 1
    assert mcf.prompt == "Question: Which is a mammal?\n A. trout\n B. otter\n C. wasp\nAnswer:"
    cf = et.build_request(et.TASKS_BY_NAME["arc_cf:easy"], line)
    assert cf.continuations == (" trout", " otter", " wasp") and "A." not in cf.prompt
    hy = et.build_request(et.TASKS_BY_NAME["arc_hybrid:easy"], line, few_shots=[line])
    assert hy.prompt.count("Question:") == 2 and "Answer: otter\n\n" in hy.prompt and hy.continuations[1] == " otter"
    wino = et.build_request(et.TASKS_BY_NAME["winogrande_cf"], {"sentence": "The cat chased the mouse because _ was hungry.", "option1": "the cat", "option2": "the mouse", "answer": "1"})
    assert wino.continuations[0] == " The cat chased the mouse because the cat was hungry." and wino.gold_idx == 0
    assert et.build_request(et.TASKS_BY_NAME["mmlu_mcf:anatomy"], {"question": "q", "choices": ["w", "x", "y", "z"], "answer": 3}).gold_idx == 3
    assert et.build_request(et.TASKS_BY_NAME["hellaswag_cf"], {"activity_label": "Cooking", "ctx_a": "A man", "ctx_b": "he", "endings": ["a", "b", "c", "d"], "label": "2"}).gold_idx == 2


def test_normalisations_pick_different_winners():
    # long continuation with a larger total but smaller per-token / per-character log-probability
    scores = et.choice_scores(logprobs=[-6.0, -4.0], continuations=[" a long answer here", " no"], num_tokens=[6, 1], unconditioned_logprobs=[-6.5, -1.0])
    assert scores["acc_token"] == [-1.0, -4.0] and scores["acc_pmi"] == [0.5, -3.0]
    acc = et.accuracy(scores, gold_idx=0)
    assert acc == {"acc_token": 1.0, "acc_char": 1.0, "acc_pmi": 1.0}
    agg = et.aggregate([{"acc_token": 1.0}, {"acc_token": 0.0}, {"acc_token": 1.0}, {"acc_token": 1.0}])
    assert abs(agg["acc_token"] - 0.75) < 1e-9 and abs(agg["acc_token_stderr"] - math.sqrt(0.25 / 4)) < 1e-9


class ByteTokenizer:
    """One token per byte (ids 1..255), enough to drive the harness."""

    bos_token_id = 0

    def encode(self, text, add_special_tokens=False):
        return [min(b, 255) for b in text.encode()]


def _scorer_run(out_file, tp, pp):
    import nanotron_b200.distributed as dist
    from nanotron_b200.eval.harness import LogLikelihoodScorer, evaluate_task
    from nanotron_b200.trainer import DistributedTrainer
    from test_distributed_cpu import _deterministic_init

    class T(DistributedTrainer):
        def _load_model_checkpoint(self, model):
            _deterministic_init(model)
            return model

    t = T(make_config(tiny_llama_config(), tp=tp, pp=pp, seq=32))
    scorer = LogLikelihoodScorer(t.unwrapped_model.model, t.parallel_context, ByteTokenizer(), max_length=64, batch_size=3)
    pairs = [("Question: 1+1?\nAnswer:", " 2"), ("Question: 1+1?\nAnswer:", " eleven"), ("Answer:", " 2"), ("A much longer context that shifts the padding of the batch", " tail"), ("x", " y")]
    got = scorer.loglikelihoods(pairs)
    task = et.TASKS_BY_NAME["arc_cf:easy"]
    lines = [{"question": f"What is {i}?", "choices": {"text": ["alpha", "beta", "gamma"], "label": ["A", "B", "C"]}, "answerKey": "ABC"[i % 3]} for i in range(4)]
    res = evaluate_task(scorer, task, lines)
    if dist.get_rank(t.parallel_context.world_pg) == 0:
        torch.save({"ll": got, "res": res}, out_file)
    dist.barrier()
    t.parallel_context.destroy()


def test_harness_matches_direct_computation_and_parallel_layouts(tmp_path):
    single = str(tmp_path / "single.pt")
    run_distributed(_scorer_run, 1, out_file=single, tp=1, pp=1)
    a = torch.load(single)
    # direct computation on one rank: full logits -> log_softmax -> gather the continuation tokens
    from helpers import single_process_env
    from nanotron_b200.trainer import DistributedTrainer
    from test_distributed_cpu import _deterministic_init

    single_process_env()

    class T(DistributedTrainer):
        def _load_model_checkpoint(self, model):
            _deterministic_init(model)
            return model

    t = T(make_config(tiny_llama_config(), seq=32))
    tok = ByteTokenizer()
    model = t.unwrapped_model.model
    model.eval()
    for (context, cont), (ll, n) in zip([("Question: 1+1?\nAnswer:", " 2"), ("Question: 1+1?\nAnswer:", " eleven")], a["ll"][:2]):
        c, k = tok.encode(context), tok.encode(cont)
        ids = torch.tensor([c + k])
        with torch.no_grad():
            logits = model(input_ids=ids, input_mask=torch.ones_like(ids, dtype=torch.bool)).float().view(ids.shape[1], -1)
        lp = torch.log_softmax(logits, -1)
        exp = sum(float(lp[len(c) + j - 1, k[j]]) for j in range(len(k)))
        assert n == len(k) and abs(ll - exp) < 1e-3, (ll, exp)
    t.parallel_context.destroy()
    assert a["res"]["num_samples"] == 4.0 and set(a["res"]) >= {"acc_token", "acc_char", "acc_pmi", "acc_token_stderr"}
    # the same numbers under tensor + pipeline parallelism
    par = str(tmp_path / "par.pt")
    run_distributed(_scorer_run, 4, out_file=par, tp=2, pp=2)
    b = torch.load(par)
    for (x, nx), (y, ny) in zip(a["ll"], b["ll"]):
        assert nx == ny and abs(x - y) < 1e-3, (a["ll"], b["ll"])
    assert a["res"] == b["res"]
