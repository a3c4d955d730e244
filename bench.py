#!/usr/bin/env python
"""Headline benchmark: BERT-base masked-LM training throughput (tokens/s) through the SameDiff API.

``python bench.py --gpus N --steps K --warmup W`` (for N > 1 launched under torchrun, one rank per
GPU) runs W untimed + K timed training steps of the BERT-base-shaped SameDiff graph
(12 layers, hidden 768, 12 heads, FFN 3072, seq 512, vocab 30522, batch 32 per GPU, Adam, bf16
compute with fp32 master weights, synthetic uniform token ids, 15 % masked positions) and prints one
JSON line.  ``value`` is timed on the device with inputs resident; ``e2e`` times the same steps
through ``sd.fit`` including the host->device copy of each step's inputs from pinned memory and a
device->host read of the loss.  ``--config`` selects the other BASELINE configurations
(``resnet50``, ``lstm``, ``mlp``, ``gradshare``); ``--impl reference`` reports why the reference
cannot run here.
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
    runner = runners.get(args.config)(args, rank, world, torch.device("cuda", local))
    sampler = ClockSampler(local)
    result = runner.run(sampler)
    if rank == 0:
        result.update({"n_gpus": world, "steps": args.steps, "warmup": args.warmup, "impl": "ours"})
        print(json.dumps(result))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
