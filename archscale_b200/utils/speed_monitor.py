"""Throughput / MFU monitor.

Reference: `lit_gpt/speed_monitor.py:21-74` (peak FLOP/s table), `:241-317` (rolling-window
throughput metrics and their names), `:392-434` (``estimate_flops``).  Differences: step time
comes from CUDA events on the training stream (device time, max over ranks) instead of the host
wall clock, and the monitor never forces a host sync on its own — the trainer hands it the
elapsed device time when it already synchronised for logging.
"""
from __future__ import annotations

import time
from collections import deque
from typing import Deque, Dict, Optional

import torch

# dense bf16 peak per device (the reference table, `lit_gpt/speed_monitor.py:21-62`)
GPU_AVAILABLE_FLOPS = {
    "b200": 2.25e15, "gb200": 2.5e15, "b100": 1.8e15,
    "h100-sxm": 0.9895e15, "h100-pcie": 0.7565e15, "h200": 0.9895e15,
    "a100": 312e12, "a10g": 125e12, "v100-sxm": 125e12, "v100-pcie": 112e12, "t4": 65e12,
}


def get_flops_available(device: Optional[torch.device] = None, dtype: torch.dtype = torch.bfloat16) -> Optional[float]:
    if not torch.cuda.is_available():
        return None
    name = torch.cuda.get_device_name(device).lower()
    for key in ("gb200", "b200", "b100", "h200"):
        if key in name:
            return GPU_AVAILABLE_FLOPS[key]
    if "h100" in name:
        return GPU_AVAILABLE_FLOPS["h100-sxm" if ("hbm3" in name or "sxm" in name) else "h100-pcie"]
    if "a100" in name:
        return GPU_AVAILABLE_FLOPS["a100"]
    return None


def flops_per_param(config, n_params: float) -> float:
    """Forward+backward FLOPs of one sequence: ``3·(2·N·T + attention)``."""
    T = config.block_size
    flops_per_token = 2 * n_params
    flops_per_seq = flops_per_token * T
    window = T if config.local_window is None or config.local_window < 0 else min(T, config.local_window)
    attn = config.n_layer * 4 * config.n_head * config.head_size * T * window
    return 3 * (flops_per_seq + attn)


def estimate_flops(config, n_params: float) -> float:
    return flops_per_param(config, n_params)


def matmul_parameter_count(model, config, include_head: bool = False, tp: int = 1, ep: int = 1) -> float:
    """Parameters that every token multiplies with, counted from the model that actually runs.

    The reference feeds ``estimate_flops`` the analytic non-embedding law (`pretrain.py:744-751`,
    `lit_gpt/config.py:232-265`), which hard-codes the 4·C MLP width; once a width is overridden
    (e.g. SwiGLU hidden 5632 instead of 8192) the law over-counts, so the MFU printed here uses this
    count instead.  Token embedding is a lookup (excluded); ``lm_head`` only with ``include_head``;
    routed experts count by the fraction ``routed_top_k / routed_experts`` a token visits.  ``tp`` /
    ``ep`` undo the physical slicing of tensor- / expert-parallel models (local shapes → whole model).
    """
    frac = 1.0
    if getattr(config, "moe", False) and config.routed_experts > 0:
        frac = config.routed_top_k / config.routed_experts
    n = 0.0
    for name, p in model.named_parameters():
        if ".wte." in name or name.startswith("wte."):
            continue
        if "lm_head" in name:
            if include_head:
                n += p.numel()
            continue
        k = float(p.numel())
        if getattr(p, "_tp_sharded", False):
            k *= tp
        if ".mods_in." in name or ".mods_out." in name:
            k *= frac * (ep if getattr(p, "_ep_local", False) else 1)
        n += k
    return n


def measured_peaks(root: Optional[str] = None) -> Dict[str, float]:
    """Roofline denominators measured on this machine (``MEASURED_PEAKS.json`` beside the package's parent
    directory) or the stated fallback (6.65 TB/s, 1.59 PFLOP/s burst, 1.4 PFLOP/s sustained)."""
    import json
    import os
    root = root or os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    out = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "kind": "fallback"}
    try:
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as fh:
            d = json.load(fh)
        for k in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
            if d.get(k):
                out[k] = float(d[k])
        out["kind"] = "measured"
    except (OSError, ValueError):
        pass
    return out


class SpeedMonitor:
    """Rolling-window throughput; call :meth:`on_train_batch_end` once per micro-batch."""

    def __init__(self, flops_available: Optional[float] = None, window_size: int = 2, world_size: int = 1,
                 log_fn=None) -> None:
        self.flops_available = flops_available
        self.world_size = world_size
        self.log_fn = log_fn
        self.hist_samples: Deque[int] = deque(maxlen=window_size + 1)
        self.hist_time: Deque[float] = deque(maxlen=window_size + 1)
        self.hist_flops: Deque[float] = deque(maxlen=window_size + 1)
        self.total_eval_time = 0.0
        self.step = -1

    def on_train_batch_end(self, samples: int, train_elapsed: float, flops_per_batch: Optional[float] = None,
                           lengths: Optional[int] = None, train_loss: Optional[float] = None) -> Dict[str, float]:
        self.step += 1
        m: Dict[str, float] = {}
        self.hist_samples.append(samples)
        self.hist_time.append(train_elapsed)
        if len(self.hist_time) == self.hist_time.maxlen:
            d_samples = self.hist_samples[-1] - self.hist_samples[0]
            d_time = max(self.hist_time[-1] - self.hist_time[0], 1e-9)
            batches = len(self.hist_samples) - 1
            dev_sps = d_samples / d_time
            m.update({
                "throughput/batches_per_sec": batches * self.world_size / d_time,
                "throughput/samples_per_sec": dev_sps * self.world_size,
                "throughput/device/batches_per_sec": batches / d_time,
                "throughput/device/samples_per_sec": dev_sps,
            })
            if lengths is not None:
                avg_len = lengths / max(samples, 1)
                m["throughput/tokens_per_sec"] = dev_sps * avg_len * self.world_size
                m["throughput/device/tokens_per_sec"] = dev_sps * avg_len
        if flops_per_batch is not None:
            self.hist_flops.append(flops_per_batch)
        if len(self.hist_flops) == self.hist_flops.maxlen:
            d_time = max(self.hist_time[-1] - self.hist_time[0], 1e-9)
            dev_fps = sum(list(self.hist_flops)[:-1]) / d_time
            m["throughput/flops_per_sec"] = dev_fps * self.world_size
            m["throughput/device/flops_per_sec"] = dev_fps
            if self.flops_available:
                m["throughput/device/mfu"] = dev_fps / self.flops_available
        m.update({"time/train": train_elapsed, "time/val": self.total_eval_time,
                  "time/total": train_elapsed + self.total_eval_time, "samples": samples})
        if lengths is not None:
            m["total_tokens"] = lengths * self.world_size
        if train_loss is not None:
            import math
            m["metric/train_loss"] = train_loss
            m["metric/train_ppl"] = math.exp(min(train_loss, 50.0))
        if self.log_fn is not None:
            self.log_fn(m, self.step)
        return m

    def eval_end(self, eval_elapsed: float) -> None:
        self.total_eval_time += eval_elapsed


class DeviceStepTimer:
    """CUDA-event timer on the current stream; ``elapsed_ms`` synchronises on the end event only."""

    def __init__(self, enabled: bool = True) -> None:
        self.enabled = enabled and torch.cuda.is_available()
        self._t0 = None
        self._start = self._end = None

    def start(self) -> None:
        if self.enabled:
            self._start = torch.cuda.Event(enable_timing=True)
            self._end = torch.cuda.Event(enable_timing=True)
            self._start.record()
        else:
            self._t0 = time.perf_counter()

    def stop(self) -> None:
        if self.enabled:
            self._end.record()
        else:
            self._t1 = time.perf_counter()

    def elapsed_ms(self) -> float:
        if self.enabled:
            self._end.synchronize()
            return self._start.elapsed_time(self._end)
        return (self._t1 - self._t0) * 1e3
