#!/usr/bin/env python
"""Headline benchmark: BERT-base masked-LM training throughput (tokens/s) through the SameDiff API.

``python bench.py --gpus N --steps K --warmup W`` (for N > 1 launched under torchrun, one rank per
GPU) runs W untimed + K timed training steps of the BERT-base-shaped SameDiff graph
(12 layers, hidden 768, 12 heads, FFN 3072, seq 512, vocab 30522, batch 32 per GPU, Adam, bf16
compute with fp32 master weights, synthetic uniform token ids, 15 % masked positions) and prints one
JSON line.  ``value`` is timed on the device with inputs resident; ``e2e`` times the same steps
through ``sd.fit`` including the host->device copy of each step's inputs from pinned memory and a
device->host read of the loss.  ``--config`` selects one other BASELINE configuration
(``resnet50``, ``lstm``, ``mlp``, ``gradshare``).  The default run measures the whole headline metric: after BERT it
times ResNet-50, the char-LSTM and the MLP (same steps / warm-up) and, for N >= 2, the gradient-exchange microbenchmark, and reports them under
``secondary`` of the same JSON line (``--no-secondary`` skips them).  For N >= 2 every runner also checks that the
replicas hold bit-identical parameters after the timed region (``replicas_equal``); a mismatch ends the run with a
non-zero exit code.  ``--impl reference`` reports why the reference cannot run here.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def _reference_arm():
    why = ("reference is a JVM/Maven project (no setup.py/pyproject; needs JDK+Maven+JavaCPP and downloads FlatBuffers at "
           "configure time): pip install of the reference tree found nothing to build")
    print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


class ClockSampler:
    """Samples SM clocks / throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._t = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20,
                 "hw_power_brake_slowdown": 0x80}
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h) if hasattr(nv, "nvmlDeviceGetCurrentClocksEventReasons") \
                    else nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for n, bit in names.items():
                    if r & bit:
                        self.reasons.add(n)
            except Exception:
                pass
            self._stop.wait(0.1)

    def start(self):
        if self.nv is not None:
            self._t = threading.Thread(target=self._run, daemon=True)
            self._t.start()

    def stop(self):
        self._stop.set()
        if self._t is not None:
            self._t.join(timeout=2)
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--config", default="bert")
    ap.add_argument("--batch", type=int, default=None, help="per-GPU batch override (debug only; invalidates the number)")
    ap.add_argument("--layers", type=int, default=None, help="layer-count override (debug only; invalidates the number)")
    ap.add_argument("--library-baseline", action="store_true", help="route ops through torch/cuBLAS + NCCL (baseline B1)")
    ap.add_argument("--mode", default="fused", help="gradient exchange for N>1: fused | nccl")
    ap.add_argument("--no-library-graphs", action="store_true", help="library baseline without CUDA-graph replay (eager launches)")
    ap.add_argument("--no-secondary", action="store_true", help="default run: BERT only (skip ResNet-50, char-LSTM, MLP and gradshare)")
    args = ap.parse_args()
    if args.impl == "reference":
        return _reference_arm()
    if args.warmup < 3:
        args.warmup = 3

    import torch
    import torch.distributed as dist
    from deeplearning4j_b200.bench import runners

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device")
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    device = torch.device("cuda", local)
    runner = runners.get(args.config)(args, rank, world, device)
    sampler = ClockSampler(local)
    result = runner.run(sampler)
    bad = result.get("replicas_equal") is False
    if args.config == "bert" and not args.no_secondary and not args.library_baseline and not args.layers and not args.batch:
        # the other half of the headline metric, measured in the same process right after BERT
        import gc
        del runner
        gc.collect()
        torch.cuda.empty_cache()
        secondary = {}
        keep = ("metric", "value", "unit", "ms_per_step", "e2e", "gpu_launches", "clocks", "config", "replicas_equal", "last_loss",
                "dtype")
        r2 = runners.get("resnet50")(args, rank, world, device).run(ClockSampler(local))
        secondary["resnet50"] = {k: r2[k] for k in keep if k in r2}
        bad = bad or r2.get("replicas_equal") is False
        gc.collect()
        torch.cuda.empty_cache()
        # the recurrent and the small dense configuration (a step is one full tBPTT sequence / one minibatch): same steps and warm-up
        for name in ("lstm", "mlp"):
            rr = runners.get(name)(args, rank, world, device).run(ClockSampler(local))
            secondary[name] = {k: rr[k] for k in keep if k in rr}
            bad = bad or rr.get("replicas_equal") is False
            del rr
            gc.collect()
            torch.cuda.empty_cache()
        if world >= 2:
            r3 = runners.get("gradshare")(args, rank, world, device).run(ClockSampler(local))
            secondary["gradshare"] = {k: r3[k] for k in ("metric", "value", "unit", "ms_per_step", "rows", "clocks", "config") if k in r3}
        result["secondary"] = secondary
    if rank == 0:
        result.update({"n_gpus": world, "steps": args.steps, "warmup": args.warmup, "impl": "ours"})
        print(json.dumps(result))
    if bad:
        if rank == 0:
            sys.stderr.write("replicas diverged: parameters differ between ranks after the timed region\n")
        if world > 1:
            dist.destroy_process_group()
        return 3
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
