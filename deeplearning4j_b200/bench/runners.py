"""Benchmark runners: each builds a model through the public API, runs warm-up + timed steps twice
(device-resident inputs, then end-to-end with pinned-host inputs and a loss read-back) and returns
the JSON fields bench.py prints."""
from __future__ import annotations

import time

import torch
import torch.distributed as dist

from ..nd.dtype import DataType
from ..ops import native, nnops


def _max_over_ranks(ms, world, device):
    if world == 1:
        return ms
    t = torch.tensor([ms], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0])


def _barrier(world):
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()


class BaseRunner:
    metric = ""
    unit = ""

    def __init__(self, args, rank, world, device):
        self.args, self.rank, self.world, self.device = args, rank, world, device
        if args.library_baseline:
            nnops.set_force_torch(True)
        else:
            native.require()

    # hooks ---------------------------------------------------------------
    def build(self): raise NotImplementedError
    def device_step(self): raise NotImplementedError        # one training step, inputs already on the device
    def e2e_step(self): raise NotImplementedError           # one step through the public API incl. H2D + loss read-back
    def work_per_step(self): raise NotImplementedError      # metric units per step per GPU
    def config(self): return {}
    def h2d_bytes(self): return 0
    def d2h_bytes(self): return 4
    def flat_params(self): return None                      # the replicated fp32 parameter buffer (replica check)
    def last_loss(self): return getattr(self, "last_loss_value", None)

    def replica_check(self):
        """After the timed region every data-parallel replica must hold bit-identical parameters: the int32 view of the
        flat fp32 buffer is summed in int64 (exact) and the sums are compared across ranks."""
        p = self.flat_params()
        if self.world == 1 or p is None:
            return None
        if isinstance(p, (list, tuple)):
            p = torch.cat([t.reshape(-1) for t in p])
        n = p.numel() // 2 * 2
        words = p.detach()[:n].view(torch.int32).to(torch.int64)
        mine = torch.stack([words.sum(), (words * (torch.arange(n, device=p.device) % 8191 + 1)).sum()])
        all_ = [torch.zeros_like(mine) for _ in range(self.world)]
        dist.all_gather(all_, mine)
        return all(bool(torch.equal(a, all_[0])) for a in all_)

    def _timed(self, fn, steps):
        _barrier(self.world)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(steps):
            fn()
        e.record()
        _barrier(self.world)
        return _max_over_ranks(s.elapsed_time(e), self.world, self.device)

    def run(self, sampler):
        a = self.args
        self.build()
        for _ in range(a.warmup):
            self.device_step()
        torch.cuda.synchronize()
        if not a.library_baseline:
            native.check_status()
        l0 = native.LAUNCHES
        sampler.start()
        ms = self._timed(self.device_step, a.steps)
        launches = native.LAUNCHES - l0
        for _ in range(2):
            self.e2e_step()
        ms_e2e = self._timed(self.e2e_step, a.steps)
        clocks = sampler.stop()
        if not a.library_baseline:
            native.check_status()
        per_step = ms / a.steps
        work = self.work_per_step() * self.world
        value = work / (per_step / 1e3)
        e2e_value = work / (ms_e2e / a.steps / 1e3)
        equal = self.replica_check()
        cfg = self.config()
        cfg["l2_policy"] = getattr(self, "l2_policy", "inputs+weights+activations per step exceed the 126 MB L2 (no explicit flush)")
        return {"metric": self.metric, "value": value, "unit": self.unit, "ms_per_step": per_step,
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": cfg, "clocks": clocks,
                "e2e": {"value": e2e_value, "unit": self.unit, "ms_per_step": ms_e2e / a.steps,
                        "h2d_bytes_per_step": self.h2d_bytes(), "d2h_bytes_per_step": self.d2h_bytes()},
                "gpu_launches": launches, "library_baseline": bool(a.library_baseline),
                "replicas_equal": equal, "last_loss": self.last_loss()}


class BertRunner(BaseRunner):
    metric = "BERT-base masked-LM training throughput"
    unit = "tokens/s"

    def build(self):
        from ..models.bert import BertConfig, build_bert_mlm
        from ..nn.updaters import Adam
        a = self.args
        self.batch = a.batch or 32
        self.seq = 512
        cfg = BertConfig.base()
        if a.layers:
            cfg.layers = a.layers
        self.cfg = cfg
        sd = build_bert_mlm(cfg, self.batch, self.seq, Adam(1e-4), DataType.BFLOAT16)
        sd.to(self.device)
        self.sd = sd
        import os
        if os.environ.get("DL4J_CUDA_GRAPHS", "1") != "0" and not (a.library_baseline and a.no_library_graphs):
            # forward + backward replay from a captured CUDA graph; the library baseline gets the same treatment so that the
            # comparison isolates the kernels from the launch overhead
            sd.getTrainingConfig().cudaGraphs = True
        g = torch.Generator().manual_seed(1234 + self.rank)
        n_tok = self.batch * self.seq
        self.n_masked = int(n_tok * 0.15) // 8 * 8
        self.n_batches = 4
        self.host, self.dev = [], []
        for _ in range(self.n_batches):
            tok = torch.randint(0, cfg.vocabSize, (self.batch, self.seq), generator=g)
            pos = torch.randperm(n_tok, generator=g)[:self.n_masked].sort().values
            lab = tok.reshape(-1)[pos].clone()
            h = {"tokens": tok.pin_memory(), "maskedPositions": pos.pin_memory(), "maskedLabels": lab.pin_memory()}
            self.host.append(h)
            self.dev.append({k: v.to(self.device) for k, v in h.items()})
        self.i = 0
        from ..samediff.training import _ensure_state
        self.state = _ensure_state(sd)
        if self.world > 1:
            from ..parallel.sharing import attach_gradient_sharing
            attach_gradient_sharing(self.state, mode="averaging", impl=("nccl" if a.library_baseline or a.mode == "nccl" else "fused"))

    def device_step(self):
        ph = self.dev[self.i % self.n_batches]
        self.i += 1
        self.state.step(ph)

    def e2e_step(self):
        ph = self.host[self.i % self.n_batches]
        self.i += 1
        hist = self.sd.fit(ph, 1)              # public API: copies inputs H2D, runs the step, reads the loss back
        self.last_loss_value = float(hist.losses[-1][-1])

    def flat_params(self):
        return self.state.flat_params

    def work_per_step(self):
        return self.batch * self.seq

    def h2d_bytes(self):
        return sum(v.numel() * v.element_size() for v in self.host[0].values())

    def config(self):
        return {"model": "SameDiff BERT-base encoder + MLM head (12 layers, hidden 768, 12 heads, FFN 3072, vocab 30522)"
                if self.cfg.layers == 12 else f"BERT {self.cfg.layers} layers (debug)",
                "global_batch": self.batch * self.world, "seq_len": self.seq, "masked_positions_per_gpu": self.n_masked,
                "updater": "Adam", "parallelism": f"dp{self.world}" + ("" if self.world == 1 else f" ({self.args.mode} gradient averaging)")}


def get(name):
    from . import runners_extra
    table = {"bert": BertRunner}
    table.update(runners_extra.TABLE)
    return table[name]
