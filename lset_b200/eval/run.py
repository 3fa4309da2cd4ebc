"""``lset-b200 eval``: run MTEB tasks on a checkpoint (cf. lset/eval/run.py:10-46)."""
from __future__ import annotations

from ..config import LSETConfig, resolve_path


def run_eval(config: LSETConfig):
    try:
        import mteb
    except ImportError as exc:
        raise SystemExit("evaluation needs the optional dependency `mteb` (pip install mteb>=2)") from exc
    from .mteb_evaluator import LSETMTEBModel

    model = LSETMTEBModel.from_pretrained(resolve_path(config.model.path), pooling=config.model.pooling,
                                          max_length=config.eval.max_length)
    names = config.eval.tasks or ["STSBenchmark"]
    tasks = mteb.get_tasks(tasks=names)
    results = mteb.evaluate(model, tasks, encode_kwargs={"batch_size": config.eval.batch_size})
    scores = {}
    for res in getattr(results, "task_results", results):
        name = getattr(res, "task_name", str(res))
        try:
            score = res.get_score()
        except Exception:
            score = None
        scores[name] = score
        print(f"{name}: main_score={score}")
    return scores
