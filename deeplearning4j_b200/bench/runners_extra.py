"""Runners for the remaining baseline configurations: ResNet-50 (ComputationGraph, Nesterovs,
threshold sharing), character LSTM (tBPTT 50), the config-1 MLP and the gradient-exchange microbenchmark."""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..nd.dtype import DataType
from .runners import BaseRunner


class _NetRunner(BaseRunner):
    sharing_mode = "shared_gradients"

    def _attach(self, net):
        if self.world > 1:
            from ..parallel.sharing import FixedThresholdAlgorithm, attach_gradient_sharing
            impl = "host" if (self.args.library_baseline or self.args.mode == "nccl") else "fused"
            if self.sharing_mode == "averaging" and impl == "host":
                impl = "nccl"
            attach_gradient_sharing(net, self.sharing_mode, impl, FixedThresholdAlgorithm(1e-3))

    def _graphs(self, net):
        """Launch-bound networks replay their forward + backward pass from a CUDA graph (the library baseline too, unless
        ``--no-library-graphs``)."""
        import os
        if os.environ.get("DL4J_CUDA_GRAPHS", "1") != "0" and not (self.args.library_baseline and self.args.no_library_graphs):
            net.setCudaGraphs(True)

    def device_step(self):
        x, y = self.dev[self.i % len(self.dev)]
        self.i += 1
        self.net.fit(x, y)

    def _issue(self, i):
        """Start the host -> device copy of batch ``i`` on the copy stream (pinned source, so it overlaps compute)."""
        if getattr(self, "_copy_stream", None) is None:
            self._copy_stream = torch.cuda.Stream()
        x, y = self.host[i % len(self.host)]
        with torch.cuda.stream(self._copy_stream):
            xd, yd = x.to(self.device, non_blocking=True), y.to(self.device, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self._copy_stream)
        return xd, yd, ev

    def e2e_step(self):
        # double-buffered input pipeline, as the framework's AsyncDataSetIterator does: the copy of the next batch is in
        # flight while this batch trains; every step still moves one full batch host -> device and reads the loss back
        if getattr(self, "_pf", None) is None:
            self._pf = self._issue(self.i)
        x, y, ev = self._pf
        self.i += 1
        self._pf = self._issue(self.i)
        cur = torch.cuda.current_stream()
        cur.wait_event(ev)
        x.record_stream(cur)
        y.record_stream(cur)
        self.net.fit(x, y)
        self.last = self.net.score()          # device -> host read of the loss
        self.last_loss_value = float(self.last)

    def flat_params(self):
        # every trainable parameter; batch-norm running statistics (kind "state") are local to a replica by design (each
        # rank normalises with the statistics of the batches it saw), so they are not part of the equality check
        net = self.net
        return [net.flat_params[e.offset:e.end] for e in net.entries if e.spec.kind != "state"]

    def h2d_bytes(self):
        return sum(t.numel() * t.element_size() for t in self.host[0])


class ResNet50Runner(_NetRunner):
    metric = "ResNet-50 training throughput"
    unit = "images/s"

    def build(self):
        from ..models.zoo import ResNet50
        from ..nn.updaters import Nesterovs
        self.batch = self.args.batch or 256
        net = ResNet50(numClasses=1000, updater=Nesterovs(0.01, 0.9), computeDataType=DataType.BFLOAT16).init(self.device)
        self.net = net
        g = torch.Generator().manual_seed(7 + self.rank)
        self.host, self.dev = [], []
        for _ in range(2):
            x = torch.randn(self.batch, 3, 224, 224, generator=g).pin_memory()
            y = torch.nn.functional.one_hot(torch.randint(0, 1000, (self.batch,), generator=g), 1000).float().pin_memory()
            self.host.append((x, y))
            self.dev.append((x.to(self.device).to(memory_format=torch.channels_last), y.to(self.device)))
        self.i = 0
        self._attach(net)
        self._graphs(net)

    def work_per_step(self):
        return self.batch

    def config(self):
        return {"model": "ResNet-50 ComputationGraph (zoo architecture, 1000 classes)", "global_batch": self.batch * self.world,
                "input": "224x224x3", "updater": "Nesterovs(0.9)", "parallelism": f"dp{self.world} threshold-encoded sharing"}


class LstmRunner(_NetRunner):
    metric = "char-LSTM training throughput"
    unit = "chars/s"

    def build(self):
        from ..models.zoo import TextGenerationLSTM
        from ..nn.updaters import Adam
        self.batch, self.T, self.vocab = self.args.batch or 64, 1000, 98
        net = TextGenerationLSTM(totalUniqueCharacters=self.vocab, hidden=1024, layers=2, tbptt=50, updater=Adam(1e-3),
                                 computeDataType=DataType.BFLOAT16).init(self.device)
        self.net = net
        g = torch.Generator().manual_seed(3 + self.rank)
        self.host, self.dev = [], []
        for _ in range(2):
            idx = torch.randint(0, self.vocab, (self.batch, self.T + 1), generator=g)
            x = torch.nn.functional.one_hot(idx[:, :-1], self.vocab).float().permute(0, 2, 1).contiguous().pin_memory()
            y = torch.nn.functional.one_hot(idx[:, 1:], self.vocab).float().permute(0, 2, 1).contiguous().pin_memory()
            self.host.append((x, y))
            self.dev.append((x.to(self.device), y.to(self.device)))
        self.i = 0
        self._attach(net)
        self._graphs(net)

    def work_per_step(self):
        return self.batch * self.T

    def config(self):
        return {"model": "2x LSTM(1024) + RnnOutput softmax, vocab 98 one-hot", "global_batch": self.batch * self.world,
                "seq_len": self.T, "tbptt": 50, "updater": "Adam", "parallelism": f"dp{self.world} threshold-encoded sharing"}


class MlpRunner(_NetRunner):
    l2_policy = ("working set of this small network (a few MB) fits in the 126 MB L2 and the timed steps run back to back, so L2 is "
                 "warm: read the number as a launch-latency figure, not a memory-bound one")
    metric = "MLP 784-512-512-10 training throughput"
    unit = "examples/s"
    sharing_mode = "shared_gradients"

    def build(self):
        from .. import nn
        self.batch = self.args.batch or 128
        conf = (nn.NeuralNetConfiguration.Builder().seed(123).updater(nn.Adam(1e-3)).list()
                .layer(nn.DenseLayer(nIn=784, nOut=512, activation="relu"))
                .layer(nn.DenseLayer(nIn=512, nOut=512, activation="relu"))
                .layer(nn.OutputLayer("MCXENT", nIn=512, nOut=10, activation="softmax")).build())
        net = nn.MultiLayerNetwork(conf)
        net.device = self.device
        self.net = net.init()
        g = torch.Generator().manual_seed(self.rank)
        x = torch.rand(self.batch, 784, generator=g).pin_memory()
        y = torch.nn.functional.one_hot(torch.randint(0, 10, (self.batch,), generator=g), 10).float().pin_memory()
        self.host, self.dev, self.i = [(x, y)], [(x.to(self.device), y.to(self.device))], 0
        self._attach(self.net)
        self._graphs(self.net)

    def work_per_step(self):
        return self.batch

    def config(self):
        return {"model": "MultiLayerNetwork MLP 784-512-512-10 fp32", "global_batch": self.batch * self.world, "updater": "Adam"}


TABLE = {"resnet50": ResNet50Runner, "lstm": LstmRunner, "mlp": MlpRunner}


class GradShareRunner(BaseRunner):
    """Gradient-exchange microbenchmark: fp32 buffers of 1 MB .. 1 GB, values N(0, 1e-3), threshold 1e-3.
    Reports, per size, the time of one fused dense step (reduce-scatter + SGD + all-gather in one kernel), one
    fused threshold step (updater + encode + exchange + decode + apply) and the NCCL all_reduce + updater baseline,
    with algorithm bandwidth (buffer bytes / time) and the achieved fraction of the NVLink roofline
    (bytes that must cross the link per GPU / 900 GB/s nominal per direction; the fraction of the measured 770 GB/s
    peer-copy bandwidth is reported beside it)."""
    metric = "gradient exchange bandwidth"
    unit = "GB/s"
    LINK_GBS = 900.0            # nominal NVLink 5 bandwidth per direction and GPU: the roofline denominator
    LINK_GBS_MEASURED = 770.0   # peer-copy bandwidth measured on this pool, reported beside it

    def run(self, sampler):
        from .. import nn
        from ..ops import native
        from ..parallel.sharing import FixedThresholdAlgorithm, attach_gradient_sharing
        W = self.world
        if W < 2:
            raise SystemExit("gradshare needs --gpus >= 2")
        sides = [512, 2048, 4096, 8192, 16384]
        rows = []
        sampler.start()
        for side in sides:
            n = side * side
            res = {"bytes": 4 * n}
            default_mm = W >= 4          # FusedSharing's own policy: in-switch reduction pays from four ranks on
            # threshold "host" = the reference's algorithm as separate launches (baseline B2): updater kernel, encode kernel,
            # NCCL all-gather of the messages, one decode launch per peer (libnd4j/include/loops/cuda/type_conversions.cu:215-354)
            for mode, impl, mm in (("averaging", "fused", None), ("averaging", "fused", not default_mm), ("averaging", "nccl", None),
                                   ("shared_gradients", "fused", None), ("shared_gradients", "host", None)):
                if impl == "host" and n > 4096 * 4096 * 4:
                    continue
                conf = (nn.NeuralNetConfiguration.Builder().seed(1).updater(nn.Sgd(0.1)).list()
                        .layer(nn.DenseLayer(nIn=side, nOut=side, hasBias=False, activation="identity"))
                        .layer(nn.LossLayer("MSE", activation="identity")).build())
                net = nn.MultiLayerNetwork(conf)
                net.device = self.device
                net.init()
                s = attach_gradient_sharing(net, mode, impl, FixedThresholdAlgorithm(1e-3), use_multimem=mm)
                g = torch.Generator(device=self.device).manual_seed(5 + self.rank)
                src = torch.randn(n, device=self.device, generator=g) * 1e-3
                if mode == "shared_gradients":
                    src = src * 10.0          # SGD lr 0.1 scales the update back to N(0, 1e-3)

                def step():
                    net.flat_grads.copy_(src)
                    if net.gradient_hook(net) is not True:
                        net._ensure_updater().update(0, 0)
                for _ in range(3):
                    step()
                torch.cuda.synchronize()
                native.check_status()
                iters = 10
                dist.barrier()
                torch.cuda.synchronize()
                ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
                for a, b in ev:
                    net.flat_grads.copy_(src)
                    a.record()
                    if net.gradient_hook(net) is not True:
                        net._ensure_updater().update(0, 0)
                    b.record()
                torch.cuda.synchronize()
                ms = sorted(a.elapsed_time(b) for a, b in ev)[iters // 2]
                t = torch.tensor([ms], dtype=torch.float64, device=self.device)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t[0])
                key = f"{'dense' if mode == 'averaging' else 'threshold'}_{impl}" + ("_alt" if mm is not None else "")
                if mm is not None:
                    res[key + "_multimem"] = bool(s.fused.use_multimem)
                res[key + "_ms"] = ms
                res[key + "_algbw_gbs"] = 4 * n / ms / 1e6
                if key == "dense_fused":
                    # per direction and GPU: reduce-scatter pulls (W-1)/W of the buffer in, all-gather receives the same again
                    link_bytes = 2 * (W - 1) / W * 4 * n
                    res["dense_fused_roofline_frac"] = (link_bytes / (self.LINK_GBS * 1e9)) / (ms / 1e3)
                    res["dense_fused_frac_of_measured_770"] = (link_bytes / (self.LINK_GBS_MEASURED * 1e9)) / (ms / 1e3)
                    res["dense_fused_multimem"] = bool(s.fused.use_multimem)
                if key == "threshold_fused":
                    link_bytes = (W - 1) * (n / 16 + 4) * 4
                    res["threshold_fused_roofline_frac"] = (link_bytes / (self.LINK_GBS * 1e9)) / (ms / 1e3)
                    # local traffic: gradient, parameters, residual read + residual, gradient written, then parameters read and written
                    res["threshold_hbm_bound_ms"] = (4 * n * 7) / 6.5475e12 * 1e3
                    res["threshold_fused_frac_of_hbm_bound"] = res["threshold_hbm_bound_ms"] / ms
                    res["threshold_fused_form"] = "bitmap" if s.fused.last_form == 1 else "index list"
                net.gradient_hook = None
                del net, s, src
                torch.cuda.empty_cache()
            rows.append(res)
        clocks = sampler.stop()
        native.check_status()
        big = rows[-1]
        return {"metric": self.metric, "value": big["dense_fused_algbw_gbs"], "unit": self.unit, "ms_per_step": big["dense_fused_ms"],
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32", "data": "synthetic",
                "config": {"model": "gradient exchange microbenchmark", "sizes_bytes": [r["bytes"] for r in rows],
                           "threshold": 1e-3, "parallelism": f"dp{W}"}, "rows": rows, "clocks": clocks,
                "gpu_launches": native.LAUNCHES}


TABLE["gradshare"] = GradShareRunner
