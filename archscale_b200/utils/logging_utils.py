"""Asynchronous metric pipeline: the training thread hands a CPU payload to a worker, hooks turn
it into ``metric/...`` scalars, the training thread drains finished results before the next
step.

Reference: `logging_utils.py:92-119,188-260` (executor, submit / drain / wait),
`:36-89` (MaxVio), `:581-828` (hooks and metric names).  The metric names are unchanged.  The
payload is built from device tensors that were *already* copied to pinned host buffers with
non-blocking copies, so building it does not stall the GPU stream (the reference calls
``.item()`` per parameter, `logging_utils.py:271-276`).
"""
from __future__ import annotations

import multiprocessing
from concurrent.futures import Future, ProcessPoolExecutor, ThreadPoolExecutor
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Sequence

import torch

ENABLE_PER_LAYER_LOGGING = True
ENABLE_PER_LAYER_EXPERT_LOGGING = False

_executor = None
_pending: List[Future] = []
logging_hooks: List[Callable] = []


def configure_logging_executor(use_multiprocessing: bool = True, max_workers: int = 1) -> None:
    global _executor
    if _executor is not None:
        _executor.shutdown(wait=False)
    if use_multiprocessing:
        _executor = ProcessPoolExecutor(max_workers=max_workers, mp_context=multiprocessing.get_context("spawn"))
    else:
        _executor = ThreadPoolExecutor(max_workers=max_workers)


def register_logging_hook(fn: Callable) -> Callable:
    logging_hooks.append(fn)
    return fn


def maxvio_batch(tokens_per_expert: torch.Tensor) -> torch.Tensor:
    """(max_i load_i − mean load) / mean load; 0 = perfectly balanced."""
    t = tokens_per_expert.float()
    if t.dim() == 2:
        t = t.mean(dim=0)
    expected = t.sum() / t.shape[0]
    return (t.max() - expected) / (expected + 1e-8)


@dataclass
class LoggingPayload:
    iter_num: int
    step_count: int
    grad_norm: float
    grad_clip: float
    param_norms: Dict[str, float] = field(default_factory=dict)
    vector_names: Sequence[str] = ()
    optimizer_stats: Dict[str, Any] = field(default_factory=dict)
    bal_loss: Optional[float] = None
    acc_seq: Optional[float] = None
    budget_loss_value: Optional[float] = None
    lc_mean_activation: Optional[float] = None
    tokens_per_expert: Optional[List[List[float]]] = None
    n_attn: Optional[List[int]] = None
    n_mlp: Optional[List[int]] = None
    lc_gate_hist: Optional[List[float]] = None
    batch_info: Optional[Dict[str, float]] = None
    attn_output_rmsnorms: Optional[List[Optional[float]]] = None
    mlp_output_rmsnorms: Optional[List[Optional[float]]] = None
    attn_outlier_pcts: Optional[List[Optional[float]]] = None
    mlp_outlier_pcts: Optional[List[Optional[float]]] = None
    attn_z_means: Optional[List[Optional[float]]] = None
    router_z_means: Optional[List[Optional[float]]] = None


@dataclass
class LoggingResult:
    step_count: int
    iter_num: int
    log_dict: Dict[str, float]
    print_lines: List[str]


def _to_float(x) -> Optional[float]:
    if x is None:
        return None
    if isinstance(x, torch.Tensor):
        return float(x.detach().float().cpu())
    return float(x)


def build_logging_payload(iter_num: int, step_count: int, grad_norm, grad_clip: float, model=None,
                          param_norms: Optional[Dict[str, Any]] = None, optimizer_stats=None, bal_loss=None,
                          batch_info=None, vector_names: Sequence[str] = ()) -> LoggingPayload:
    """Collect scalars on the host.  Call only on logging steps (it synchronises once)."""
    p = LoggingPayload(iter_num=iter_num, step_count=step_count, grad_norm=_to_float(grad_norm) or 0.0,
                       grad_clip=grad_clip, vector_names=tuple(vector_names),
                       optimizer_stats=dict(optimizer_stats or {}), bal_loss=_to_float(bal_loss),
                       batch_info=batch_info)
    if param_norms:
        names = list(param_norms)
        vals = torch.stack([torch.as_tensor(param_norms[n]).float().reshape(()) for n in names]).cpu().tolist()
        p.param_norms = dict(zip(names, vals))
    if model is not None:
        tpe = getattr(model, "tokens_per_expert", None)
        if tpe:
            p.tokens_per_expert = [t.float().cpu().tolist() for t in tpe if t is not None]
            p.n_attn, p.n_mlp = getattr(model, "n_attn", None), getattr(model, "n_mlp", None)
        for key in ("attn_output_rmsnorms", "mlp_output_rmsnorms", "attn_outlier_pcts", "mlp_outlier_pcts",
                    "attn_z_means", "router_z_means"):
            vals = getattr(model, key, None)
            if vals:
                setattr(p, key, [_to_float(v) for v in vals])
        hist = getattr(model, "lc_gate_hist", None)
        if hist:
            p.lc_gate_hist = [float((g > 0.5).float().mean().cpu()) for g in hist]
    return p


def logging_train(payload: LoggingPayload) -> LoggingResult:
    log = {
        "metric/grad_norm": payload.grad_norm,
        "metric/grad_norm_clip_ratio": payload.grad_norm / payload.grad_clip if payload.grad_clip > 0 else float("inf"),
    }
    lines: List[str] = []
    for hook in logging_hooks:
        hook(payload, log, lines)
    return LoggingResult(payload.step_count, payload.iter_num, log, lines)


def submit_logging_task(payload: LoggingPayload) -> None:
    if _executor is None:
        configure_logging_executor(use_multiprocessing=False)
    _pending.append(_executor.submit(logging_train, payload))


def drain_logging_queue(log_fn: Callable[[Dict[str, float], int], None], print_fn: Callable[[str], None] = print) -> None:
    """Emit every finished result (exceptions of the worker are re-raised here)."""
    still = []
    for fut in _pending:
        if fut.done():
            res = fut.result()
            log_fn(res.log_dict, res.step_count)
            for line in res.print_lines:
                print_fn(line)
        else:
            still.append(fut)
    _pending[:] = still


def wait_for_logging_tasks(log_fn, print_fn=print) -> None:
    for fut in list(_pending):
        fut.result()
    drain_logging_queue(log_fn, print_fn)


def shutdown() -> None:
    global _executor
    if _executor is not None:
        _executor.shutdown(wait=True)
        _executor = None


# ------------------------------------------------------------------ hooks
@register_logging_hook
def _core_metric_hook(p: LoggingPayload, log: Dict[str, float], lines: List[str]) -> None:
    if p.budget_loss_value is not None:
        log["metric/lc_budget_loss"] = p.budget_loss_value
        log["metric/lc_mean_activation"] = p.lc_mean_activation
    if p.bal_loss is not None:
        log["metric/bal_loss"] = p.bal_loss
    if p.acc_seq is not None:
        log["metric/acc_seq"] = p.acc_seq
    w2 = v2 = 0.0
    for name, norm in p.param_norms.items():
        n = name.lower()
        if "weight" in n and not any(nd in n for nd in p.vector_names):
            w2 += norm ** 2
        else:
            v2 += norm ** 2
    st = p.optimizer_stats
    if st.get("betas") is not None:
        log["metric/optimizer_beta1"], log["metric/optimizer_beta2"] = st["betas"]
    if st.get("eps") is not None:
        log["metric/optimizer_eps"] = st["eps"]
    wlr, vlr, wd = st.get("weight_lr", 0.0), st.get("vector_lr", 0.0), st.get("weight_decay", 0.0)
    log.update({"metric/weight_grad_norm": w2 ** 0.5, "metric/vector_grad_norm": v2 ** 0.5,
                "metric/intrinsic_learning_rate": wd * wlr, "metric/weight_learning_rate": wlr,
                "metric/vector_learning_rate": vlr, "metric/optimizer_weight_decay": wd})
    if st.get("non_embed_vector_lr") is not None:
        log["metric/non_embed_vector_learning_rate"] = st["non_embed_vector_lr"]


@register_logging_hook
def _expert_load_hook(p: LoggingPayload, log: Dict[str, float], lines: List[str]) -> None:
    if p.tokens_per_expert is None or p.n_attn is None or p.n_mlp is None:
        return
    all_mv = []
    for i, n_tokens in enumerate(p.tokens_per_expert):
        total = sum(n_tokens)
        if total == 0:
            continue
        if ENABLE_PER_LAYER_EXPERT_LOGGING:
            a, m = p.n_attn[i], p.n_mlp[i]
            log[f"metric/loop_{i}_attn_load"] = sum(n_tokens[:a]) / total
            log[f"metric/loop_{i}_mlp_load"] = sum(n_tokens[a:a + m]) / total
            log[f"metric/loop_{i}_skip_load"] = sum(n_tokens[a + m:]) / total
            for j, t in enumerate(n_tokens):
                log[f"metric/loop_{i}_expert_{j}_load"] = t / total
        mv = float(maxvio_batch(torch.tensor(n_tokens, dtype=torch.float32)))
        if ENABLE_PER_LAYER_LOGGING:
            log[f"metric/loop_{i}_maxvio_batch"] = mv
        all_mv.append(mv)
    if all_mv:
        log["metric/maxvio_batch_avg"] = sum(all_mv) / len(all_mv)


@register_logging_hook
def _lc_sparsity_hook(p: LoggingPayload, log: Dict[str, float], lines: List[str]) -> None:
    if not p.lc_gate_hist:
        return
    for i, s in enumerate(p.lc_gate_hist):
        if ENABLE_PER_LAYER_LOGGING:
            log[f"metric/train_sparsity_layer_{i}"] = s
    log["metric/train_sparsity_mean"] = sum(p.lc_gate_hist) / len(p.lc_gate_hist)


@register_logging_hook
def _batch_ramp_hook(p: LoggingPayload, log: Dict[str, float], lines: List[str]) -> None:
    if not p.batch_info:
        return
    for k in ("grad_accum_steps", "effective_batch_size", "batch_multiplier", "batch_ratio"):
        if k in p.batch_info:
            log[f"metric/{k}"] = p.batch_info[k]


def _per_layer(log: Dict[str, float], vals: Optional[List[Optional[float]]], stem: str) -> None:
    if not vals:
        return
    good = [(i, v) for i, v in enumerate(vals) if v is not None]
    if not good:
        return
    if ENABLE_PER_LAYER_LOGGING:
        for i, v in good:
            log[f"metric/{stem}_layer_{i}"] = v
    log[f"metric/{stem}_mean"] = sum(v for _, v in good) / len(good)


@register_logging_hook
def _activation_stats_hook(p: LoggingPayload, log: Dict[str, float], lines: List[str]) -> None:
    _per_layer(log, p.attn_output_rmsnorms, "attn_output_rmsnorm")
    _per_layer(log, p.mlp_output_rmsnorms, "mlp_output_rmsnorm")
    _per_layer(log, p.attn_outlier_pcts, "attn_outlier_pct")
    _per_layer(log, p.mlp_outlier_pcts, "mlp_outlier_pct")
    _per_layer(log, p.attn_z_means, "attn_z")
    _per_layer(log, p.router_z_means, "router_z")


class MetricLogger:
    """Sink for metrics: JSON-lines file always; W&B / MLflow when importable and requested."""

    def __init__(self, out_dir: Optional[str], project: Optional[str] = None, name: Optional[str] = None,
                 use_wandb: bool = False, use_mlflow: bool = False, rank: int = 0) -> None:
        self.rank, self._fh, self._wandb, self._mlflow = rank, None, None, None
        if rank != 0:
            return
        if out_dir:
            import os
            os.makedirs(out_dir, exist_ok=True)
            self._fh = open(os.path.join(out_dir, "metrics.jsonl"), "a")
        if use_wandb:
            try:
                import wandb
                self._wandb = wandb.init(project=project, name=name)
            except Exception as e:  # noqa: BLE001
                print(f"[logging] wandb unavailable ({e}); metrics go to metrics.jsonl only")
        if use_mlflow:
            try:
                import mlflow
                self._mlflow = mlflow
            except Exception as e:  # noqa: BLE001
                print(f"[logging] mlflow unavailable ({e})")

    def log_hyperparams(self, hp: Dict[str, Any]) -> None:
        self.log_dict({f"hparams/{k}": v for k, v in hp.items() if isinstance(v, (int, float))}, 0)

    def log_dict(self, metrics: Dict[str, float], step: int) -> None:
        if self.rank != 0:
            return
        if self._fh is not None:
            import json
            self._fh.write(json.dumps({"step": step, **{k: v for k, v in metrics.items()}}) + "\n")
            self._fh.flush()
        if self._wandb is not None:
            self._wandb.log(metrics, step=step)
        if self._mlflow is not None:
            self._mlflow.log_metrics({k.replace("@", "_at_"): v for k, v in metrics.items()}, step=step)

    def close(self) -> None:
        if self._fh is not None:
            self._fh.close()
