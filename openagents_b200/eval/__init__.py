"""Checkpoint evaluation: scorers over a serving backend, evaluation packs with metric gates, the continue / hold / rollback
decision and its evidence record."""
from .pack import EvalPack, MetricGate, decide, eval_run_evidence, run_pack  # noqa: F401
from .scorers import exact_match, multiple_choice, perplexity  # noqa: F401
