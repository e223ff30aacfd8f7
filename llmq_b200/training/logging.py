"""Training-run logger: console lines plus a JSON-array log file, one object per line.

Line kinds and fields follow the reference's TrainingRunLogger (src/training/logging.cpp) so that its tools
(wandb export, plotting) read these logs: ``cmd, option, gpu-model, dataset, allocator, sol, step, eval, gpu,
info, abs-maxes``.  Only rank 0 writes.  A per-line callback receives every JSON object (live export).
"""
from __future__ import annotations

import datetime
import enum
import json
import os
import sys
from typing import Callable, Optional


class LogVerbosity(enum.IntEnum):
    SILENT = -2
    QUIET = -1
    DEFAULT = 0
    VERBOSE = 1


def _now() -> str:
    return datetime.datetime.now().isoformat(sep=" ", timespec="milliseconds")


def format_tps(tokens: int, ms: float) -> str:
    if ms <= 0:
        return "-"
    tps = int(1000 * tokens / ms)
    return f"{tps:5d}" if tps < 100_000 else f"{tps // 1000:4d}k"


def format_time(ms: float) -> str:
    ms = int(ms)
    return f"{ms // 1000:5d}  s" if ms >= 100_000 else f"{ms:5d} ms"


class TrainingRunLogger:
    def __init__(self, file_name: Optional[str], callback: Optional[Callable[[dict], None]] = None,
                 verbosity: LogVerbosity = LogVerbosity.DEFAULT, rank: int = 0, final_step: int = -1):
        self.rank, self.verbosity, self.callback = rank, int(verbosity), callback
        self.final_step = final_step
        self.expected_ns_per_token = 0.0
        self._sum_loss, self._n_loss = 0.0, 0
        self._first = True
        self._f = None
        if rank == 0 and file_name:
            os.makedirs(os.path.dirname(os.path.abspath(file_name)), exist_ok=True)
            self._f = open(file_name, "w")
            self._f.write("[\n")
        self.file_name = file_name

    # ------------------------------------------------------------------ plumbing
    def _line(self, obj: dict) -> None:
        if self.rank != 0:
            return
        obj = {"log": obj.pop("log"), "time": _now(), **obj}
        if self._f:
            self._f.write(("  " if self._first else ",\n  ") + json.dumps(obj))
            self._first = False
            self._f.flush()
        if self.callback:
            self.callback(obj)

    def _print(self, level: int, msg: str) -> None:
        if self.rank == 0 and self.verbosity >= level:
            print(msg)
            sys.stdout.flush()

    def close(self) -> None:
        if self._f:
            self._f.write("\n]\n")
            self._f.close()
            self._f = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    # ------------------------------------------------------------------ start-up blocks
    def log_cmd(self, argv) -> None:
        self._line({"log": "cmd", "cmd": list(argv)})

    def log_options(self, options: dict) -> None:
        for k, v in options.items():
            self._line({"log": "option", "name": k, "value": v if isinstance(v, (int, float, bool, str, type(None))) else str(v)})
        if options:
            width = max(len(k) for k in options)
            self._print(0, "[Options]\n" + "\n".join(f"  {k:<{width}}: {v}" for k, v in options.items()) + "\n")

    def log_gpu_model(self, rank: int, name: str, mem_total: int, mem_reserved: int = 0, extra: Optional[dict] = None) -> None:
        self._line({"log": "gpu-model", "rank": rank, "name": name, "memory": mem_total, "reserved": mem_reserved, **(extra or {})})
        self._print(0, f"[System {rank}]\n  {name}, {mem_total / 2**30:.1f} GiB\n")

    def log_dataset(self, train_loader, eval_loader=None) -> None:
        d = {"log": "dataset", "train_files": train_loader.num_files, "train_tokens": train_loader.num_tokens,
             "train_chunks": train_loader.num_chunks, "seq_len": train_loader.seq_len}
        if eval_loader is not None:
            d.update({"eval_files": eval_loader.num_files, "eval_tokens": eval_loader.num_tokens, "eval_chunks": eval_loader.num_chunks})
        self._line(d)
        self._print(0, f"[Dataset]\n  train: {d['train_tokens'] / 1e6:.1f}M tokens in {d['train_files']} files"
                    + (f"\n  eval : {d['eval_tokens'] / 1e6:.1f}M tokens in {d['eval_files']} files" if eval_loader is not None else "") + "\n")

    def log_allocator(self, report_or_trainer, gpu_id: int = 0) -> None:
        rep = report_or_trainer.get_allocator_info(gpu_id) if hasattr(report_or_trainer, "get_allocator_info") else report_or_trainer
        self._line({"log": "allocator", "gpu": gpu_id, "stats": rep})
        lines = [f"[Allocator State {gpu_id}]"]
        for k, v in rep.items():
            if k.startswith("_"):
                continue
            lines.append(f"  {k:<12}: device {v['device'] / 2**20:9.0f} MiB | pinned {v['pinned'] / 2**20:9.0f} MiB | host {v['host'] / 2**20:7.0f} MiB")
        if "_stack" in rep:
            st = rep["_stack"]
            top = sorted(st.get("breakdown", {}).items(), key=lambda kv: -kv[1])[:4]
            lines.append(f"  Stack high-water {st['high_water'] / 2**20:.0f} MiB of {st['capacity'] / 2**20:.0f} MiB"
                         + (" (" + ", ".join(f"{k} {v / 2**20:.0f}" for k, v in top) + ")" if top else ""))
        if "_device" in rep:
            d = rep["_device"]
            lines.append(f"  Free {d['free'] / 2**20:.0f} MiB | Reserved {d['reserved'] / 2**20:.0f} MiB | Total {d['total'] / 2**20:.0f} MiB")
        self._print(0, "\n".join(lines) + "\n")

    def log_sol_estimate(self, ns_per_token_spec: float, ns_per_token_measured: float = 0.0, measured_peak_tflops: float = 0.0,
                         spec_peak_tflops: float = 0.0) -> None:
        self.expected_ns_per_token = ns_per_token_spec
        self._line({"log": "sol", "ns_per_token": ns_per_token_spec, "ns_per_token_measured_peak": ns_per_token_measured,
                    "measured_bf16_tflops": measured_peak_tflops, "spec_bf16_tflops": spec_peak_tflops})
        msg = f"[Speed of Light]\n  {ns_per_token_spec:.1f} ns/token at spec-sheet peak"
        if ns_per_token_spec > 0:
            msg += f" ({1e9 / ns_per_token_spec / 1e3:.1f}k tok/s)"
        if measured_peak_tflops > 0 and spec_peak_tflops > 0:
            msg += f"\n  Benchmark: {100 * measured_peak_tflops / spec_peak_tflops:.0f}% of spec sheet ({measured_peak_tflops:.0f} TFLOP/s bf16)"
        self._print(0, msg + "\n")

    def set_expected_time_per_token(self, trainer_or_ns) -> None:
        if isinstance(trainer_or_ns, (int, float)):
            self.expected_ns_per_token = float(trainer_or_ns)
            return
        from ..utils.sol import estimate_speed_of_light
        tr = trainer_or_ns
        opts = tr.options
        self.expected_ns_per_token = estimate_speed_of_light(tr.config, tr.seq_length, opts.model_type or tr.config.dtype, opts.matmul_dtype(),
                                                             tr.world_size)

    # ------------------------------------------------------------------ per-step lines
    def log_step(self, step: int, step_tokens: int, duration_ms: float, norm: float, loss: float, loss_1k: float = 0.0,
                 lse_max: float = 0.0, lse_mean: float = 0.0, lr: float = 0.0) -> None:
        self._sum_loss += loss
        self._n_loss += 1
        progress = 100.0 * step / self.final_step if self.final_step > 0 else 0.0
        sol = ""
        if self.expected_ns_per_token > 0 and duration_ms > 0:
            peak_ms = self.expected_ns_per_token * step_tokens / 1e6
            sol = f" | sol {100.0 * peak_ms / duration_ms:.1f}%"
        self._print(0, f"[T] step {step:5d} [{progress:4.1f}%] | time: {format_time(duration_ms)} | norm {norm:10f} | loss {loss:10f} "
                       f"| tps {format_tps(step_tokens, duration_ms)}{sol}")
        self._line({"log": "step", "step": step, "step_tokens": step_tokens, "duration_ms": duration_ms, "norm": norm, "loss": loss,
                    "lr": lr, "lse_max": lse_max, "lse_mean": lse_mean, "loss_1k": loss_1k})

    def log_eval(self, step: int, eval_tokens: int, duration_ms: float, loss: float, loss_1k: float = 0.0) -> None:
        progress = 100.0 * step / self.final_step if self.final_step > 0 else 0.0
        train_avg = self._sum_loss / max(1, self._n_loss)
        self._print(-1, f"\x1b[1m[V] step {step:5d} [{progress:4.1f}%] | time: {format_time(duration_ms)} | eval {loss:10f} | train {train_avg:9f} "
                        f"| tps {format_tps(eval_tokens, duration_ms)}\x1b[22m")
        self._sum_loss, self._n_loss = 0.0, 0
        self._line({"log": "eval", "step": step, "eval_tokens": eval_tokens, "duration_ms": duration_ms, "loss": loss, "loss_1k": loss_1k})

    def log_gpu_state(self, step: int, gpu_id: int, info) -> None:
        d = info.to_dict() if hasattr(info, "to_dict") else dict(info)
        self._line({"log": "gpu", "step": step, "id": gpu_id, "clock": d.get("clock"), "max_clock": d.get("max_clock"), "fan": d.get("fan"),
                    "power": d.get("power"), "power_limit": d.get("power_limit"), "temperature": d.get("temperature"),
                    "temp_slowdown": d.get("temp_slowdown"), "gpu_util": d.get("gpu_utilization"), "mem_util": d.get("mem_utilization"),
                    "throttle": d.get("throttle_reason"), "dram_free": d.get("mem_free"), "pcie_rx": d.get("pcie_rx"), "pcie_tx": d.get("pcie_tx")})
        self._print(1, f"[G] step {step:5d} [gpu {gpu_id:2d}] | power {int((d.get('power') or 0) / 1000):4d} W   | temp {d.get('temperature', 0):3d} "
                       f"/{d.get('temp_slowdown', 0):3d}°C | clock {d.get('clock', 0):4d} MHz")

    def log_message(self, step: int, message: str) -> None:
        self._line({"log": "info", "step": step, "message": message})
        self._print(0, f"[I] step {step:5d} | {message}")

    def log_time_breakdown(self, step: int, breakdown: dict) -> None:
        self._line({"log": "info", "step": step, "time-breakdown": breakdown})
        self._print(0, "[I] " + " | ".join(f"{k} {v:.1f} ms" for k, v in breakdown.items()))

    def log_abs_maxes(self, step: int, values: dict) -> None:
        self._line({"log": "abs-maxes", "step": step, "values": values})
