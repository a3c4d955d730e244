"""Worker for the multi-GPU tests (launched by torchrun, one rank per GPU): fused NVLink kernels against
the NCCL / host-codec paths, and a bounded-wait timeout check."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


# classes of the test network; 16 gives a parameter count on the 16-byte grid, 10 puts Adam's second state half 8 bytes off it
N_OUT = int(os.environ.get("DL4J_TEST_NOUT", "16"))


def make_net(rank, updater, bf16):
    from deeplearning4j_b200 import nn, DataType
    b = nn.NeuralNetConfiguration.Builder().seed(100 + rank).updater(updater).l2(1e-4)
    if bf16:
        b.computeDataType(DataType.BFLOAT16)
    conf = (b.list().layer(nn.DenseLayer(nIn=256, nOut=512, activation="relu"))
            .layer(nn.DenseLayer(nIn=512, nOut=264, activation="tanh"))
            .layer(nn.OutputLayer("MCXENT", nIn=264, nOut=N_OUT, activation="softmax")).build())
    net = nn.MultiLayerNetwork(conf)
    net.device = torch.device("cuda", torch.cuda.current_device())
    return net.init()


def data(rank, step):
    g = torch.Generator().manual_seed(1000 * rank + step)
    x = torch.rand(64, 256, generator=g).cuda()
    y = torch.nn.functional.one_hot(torch.randint(0, N_OUT, (64,), generator=g), N_OUT).float().cuda()
    return x, y


def gather_equal(t, tol=0.0):
    world = dist.get_world_size()
    out = [torch.zeros_like(t) for _ in range(world)]
    dist.all_gather(out, t.contiguous())
    return all(float((out[0] - o).abs().max()) <= tol for o in out)


def run_pair(mode, updater_fn, bf16, multimem, steps=6, form=None, tau=1e-3):
    from deeplearning4j_b200.parallel.sharing import attach_gradient_sharing, FixedThresholdAlgorithm
    from deeplearning4j_b200.parallel import codec
    from deeplearning4j_b200.ops import native
    rank = dist.get_rank()
    a, b = make_net(rank, updater_fn(), bf16), make_net(rank, updater_fn(), bf16)
    sa = sb = None
    if mode == "averaging":
        attach_gradient_sharing(a, "averaging", "fused", use_multimem=multimem)
        attach_gradient_sharing(b, "averaging", "nccl")
    else:
        sa = attach_gradient_sharing(a, "shared_gradients", "fused", FixedThresholdAlgorithm(tau))
        if form is None:
            sb = attach_gradient_sharing(b, "shared_gradients", "host", FixedThresholdAlgorithm(tau))
            sa.encoding = sb.encoding = codec.BITMAP_ENCODING
        else:
            # index-list / automatic form against the bitmap form of the same kernel (itself checked against the host codec):
            # what is sent when differs, the conserved quantity (parameters minus all unsent residuals) must not
            sb = attach_gradient_sharing(b, "shared_gradients", "fused", FixedThresholdAlgorithm(tau))
            sb.encoding = codec.BITMAP_ENCODING
            sa.encoding = None if form == -1 else form
    assert torch.equal(a.flat_params, b.flat_params)
    for st in range(steps):
        x, y = data(rank, st)
        if mode != "averaging" and form is not None:
            # the two runs send different things at different times, so their parameters (and with them the gradients of a
            # real model) drift apart; a gradient sequence that does not depend on the parameters keeps the conserved
            # quantity comparable
            gg = torch.Generator(device="cuda").manual_seed(77 * rank + st)
            grad = torch.randn(a.flat_grads.numel(), device="cuda", generator=gg) * (0.8 * tau)
            for net_ in (a, b):
                net_.flat_grads.copy_(grad)
                assert net_.gradient_hook(net_) is True
            continue
        a.fit(x, y)
        b.fit(x, y)
        if st == 0 and mode != "averaging" and not bf16 and form is None:
            # from identical parameters and empty residuals one step must agree exactly (same messages)
            mism = int((a.flat_params != b.flat_params).sum())
            assert mism <= 2, ("first threshold step differs", mism)
    torch.cuda.synchronize()
    native.check_status()
    tol = 2e-2 if bf16 else 2e-5
    d = float((a.flat_params - b.flat_params).abs().max())
    if mode == "averaging":
        assert d <= tol, (mode, bf16, multimem, d)
    else:
        # Elements whose accumulated update sits exactly at the threshold may be sent one step earlier or later
        # by the two implementations (last-bit differences in the updater math); what must agree is the quantity
        # the protocol conserves: parameters minus the sum of every rank's unsent residual.
        ra, rb = sa.fused.residual.clone(), (sb.fused.residual if hasattr(sb, "fused") else sb.residual).clone()
        dist.all_reduce(ra); dist.all_reduce(rb)
        inv = float(((a.flat_params - ra) - (b.flat_params - rb)).abs().max())
        assert inv <= (5e-3 if bf16 else 5e-4), (mode, bf16, inv)
        if form is None:
            assert d <= 8 * tau, (mode, bf16, d)
            assert float((a.flat_params - b.flat_params).abs().mean()) <= 0.3 * tau
        else:
            assert d <= 6 * tau, (mode, bf16, form, d)        # a value is at most a few thresholds behind in either form
        if form == codec.FLEXIBLE_ENCODING:
            # the index list really was used, and the density feedback arrived
            assert sa.fused.last_form == 0
            assert sa.fused._poll_sent(wait=True) is not None
    assert gather_equal(a.flat_params), "fused replicas diverged"
    if a.flat_shadow is not None:
        assert gather_equal(a.flat_shadow.float())
        ref = a.flat_params.clone()
        for e, so in zip(a.entries, a.shadow_offsets):
            sh = a.flat_shadow[so:so + e.spec.numel].float()
            assert float((sh - ref[e.offset:e.end]).abs().max()) <= 1e-2
    assert float(a.flat_grads.abs().max()) == 0.0
    return d


def bucketed_case(graphs, updater_fn, buckets=5, steps=7):
    """SameDiff BERT-shaped model: exchange overlapped with backward bucket by bucket (fused kernels on a side stream, optionally
    inside the captured CUDA graph) against NCCL all-reduce + the local updater."""
    from deeplearning4j_b200 import DataType
    from deeplearning4j_b200.models.bert import BertConfig, build_bert_mlm
    from deeplearning4j_b200.ops import native
    from deeplearning4j_b200.parallel.fused import BucketedAveraging
    from deeplearning4j_b200.parallel.sharing import attach_gradient_sharing
    from deeplearning4j_b200.samediff.training import _ensure_state
    rank = dist.get_rank()
    dev = torch.device("cuda", torch.cuda.current_device())
    cfg = BertConfig(vocabSize=512, hidden=128, layers=3, heads=4, ffn=256, maxPositions=64)
    B, T = 4, 64
    states = []
    for impl in ("fused", "nccl"):
        torch.manual_seed(7)
        sd = build_bert_mlm(cfg, B, T, updater_fn(), DataType.BFLOAT16).to(dev)
        sd.getTrainingConfig().cudaGraphs = bool(graphs)
        st = _ensure_state(sd)
        hook = attach_gradient_sharing(st, "averaging", impl, buckets=buckets)
        states.append((sd, st, hook))
    (sda, a, ha), (sdb, b, hb) = states
    assert isinstance(ha, BucketedAveraging) and ha.n_buckets >= 3, type(ha)
    assert torch.equal(a.flat_params, b.flat_params)
    for step in range(steps):
        g = torch.Generator().manual_seed(50 * rank + step)
        tok = torch.randint(0, cfg.vocabSize, (B, T), generator=g)
        pos = torch.randperm(B * T, generator=g)[:40].sort().values
        ph = {"tokens": tok.to(dev), "maskedPositions": pos.to(dev), "maskedLabels": tok.reshape(-1)[pos].to(dev)}
        la = a.step(ph)
        lb = b.step(ph)
    torch.cuda.synchronize()
    native.check_status()
    d = float((a.flat_params - b.flat_params).abs().max())
    assert d <= 3e-2, ("bucketed vs nccl", graphs, d)
    assert abs(float(la) - float(lb)) <= 5e-2 * max(1.0, abs(float(lb))), (float(la), float(lb))
    assert gather_equal(a.flat_params), "bucketed replicas diverged"
    assert gather_equal(a.flat_shadow.float())
    for e, so in zip(a.entries, a.shadow_offsets):
        sh = a.flat_shadow[so:so + e.spec.numel].float()
        assert float((sh - a.flat_params[e.offset:e.end]).abs().max()) <= 1e-2, e.spec.name
    assert float(a.flat_grads.abs().max()) == 0.0
    early = sum(1 for c in getattr(ha, "fired_early", []) if c)
    return d, ha.n_buckets, early


def param_average_case(bf16, steps=7, freq=3):
    """ParallelWrapper AVERAGING with averagingFrequency 3: the fused parameter-averaging kernel against the library all-reduce path
    (same data per rank, so the two wrappers must stay equal up to summation order) and equal replicas after an averaging step."""
    from deeplearning4j_b200 import nn
    from deeplearning4j_b200.ops import native
    from deeplearning4j_b200.parallel.wrapper import ParallelWrapper, TrainingMode
    rank = dist.get_rank()
    a, b = make_net(rank, nn.Adam(1e-3), bf16), make_net(rank, nn.Adam(1e-3), bf16)
    wa = ParallelWrapper.Builder(a).workers(dist.get_world_size()).trainingMode(TrainingMode.AVERAGING).averagingFrequency(freq).build()
    wb = ParallelWrapper(b, workers=dist.get_world_size(), trainingMode=TrainingMode.AVERAGING, averagingFrequency=freq, impl="nccl") \
        if "impl" in ParallelWrapper.__init__.__code__.co_varnames else None
    assert getattr(wa, "_fused_avg", None) is not None, "the fused averaging path was not taken"
    if wb is not None:
        assert getattr(wb, "_fused_avg", None) is None
        assert torch.equal(a.flat_params, b.flat_params)
    worst = 0.0
    for step in range(steps):
        x, y = data(rank, step)
        a.fit(x, y)
        if wb is not None:
            b.fit(x, y)
            worst = max(worst, float((a.flat_params - b.flat_params).abs().max()))
        if (step + 1) % freq == 0:
            torch.cuda.synchronize()
            assert gather_equal(a.flat_params), f"replicas differ after the averaging step {step}"
            if a.flat_shadow is not None:
                ref = a.flat_shadow.float()
                assert gather_equal(ref)
        elif step % freq == 0 and step > 0:
            assert not gather_equal(a.flat_params), "replicas should drift between averaging steps (different data per rank)"
    torch.cuda.synchronize()
    native.check_status()
    assert worst < 2e-6, worst
    return worst


def timeout_case():
    """Rank 1 skips a step: rank 0's peer wait must expire and report through the status word, leaving the
    context usable."""
    from deeplearning4j_b200 import nn
    from deeplearning4j_b200.parallel.sharing import attach_gradient_sharing
    from deeplearning4j_b200.ops import native
    rank = dist.get_rank()
    net = make_net(rank, nn.Sgd(0.1), False)
    attach_gradient_sharing(net, "averaging", "fused", use_multimem=False)
    x, y = data(rank, 0)
    net.fit(x, y)
    torch.cuda.synchronize()
    native.check_status()
    dist.barrier()
    if rank == 0:
        net.fit(x, y)                   # nobody answers
        torch.cuda.synchronize()
        try:
            native.check_status()
            raised = False
        except RuntimeError as e:
            raised = "peer wait" in str(e)
        assert raised, "bounded peer wait did not report a timeout"
        z = torch.ones(8, device="cuda").sum().item()     # context still usable
        assert z == 8.0
    dist.barrier()


def main():
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from deeplearning4j_b200 import nn
    what = sys.argv[1] if len(sys.argv) > 1 else "all"
    res = {}
    if what in ("all", "averaging"):
        for upd in (lambda: nn.Adam(1e-3), lambda: nn.Nesterovs(0.05, 0.9)):
            for bf16 in (False, True):
                for mm in (False, True):
                    res[("avg", upd().JAVA, bf16, mm)] = run_pair("averaging", upd, bf16, mm)
    if what in ("all", "threshold"):
        for bf16 in (False, True):
            # plain SGD: the update is a smooth function of the gradient, so the two implementations stay comparable
            res[("thr", bf16)] = run_pair("threshold", lambda: nn.Sgd(0.5), bf16, False)
            # index-list form at a low density (the list of a chunk holds one entry per 16 elements)
            res[("thr-list", bf16)] = run_pair("threshold", lambda: nn.Sgd(0.5), bf16, False, form=0, tau=4e-3)
        # form chosen from the reported density, with an updater that has state
        res[("thr-auto",)] = run_pair("threshold", lambda: nn.Nesterovs(0.05, 0.9), True, False, form=-1, tau=2e-3)
    if what in ("all", "bucketed"):
        for graphs in (False, True):
            for upd in (lambda: nn.Adam(1e-3), lambda: nn.Nesterovs(0.05, 0.9)):
                res[("bucketed", graphs, upd().JAVA)] = bucketed_case(graphs, upd)
    if what in ("all", "paramavg"):
        for bf16 in (False, True):
            res[("paramavg", bf16)] = param_average_case(bf16)
    if what == "timeout":
        timeout_case()
    if dist.get_rank() == 0:
        print("RESULT", {str(k): v for k, v in res.items()})
        print("WORKER_OK")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
