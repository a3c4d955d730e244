"""Word2vec batch kernel and the t-SNE edge-force kernel against the step-by-step torch formulation of the same ops."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _tables(V, D, seed):
    g = torch.Generator().manual_seed(seed)
    return ((torch.rand(V, D, generator=g) - 0.5), (torch.rand(V, D, generator=g) - 0.5), (torch.rand(V, D, generator=g) - 0.5))


@pytest.mark.parametrize("D", [24, 100, 300])
def test_skipgram_kernel_matches_the_sequential_formulation(D):
    """Single examples (one launch each) are order-free, so the kernel and the sequential op must agree to rounding; both the
    hierarchical-softmax and the negative-sampling branch run, with the sample sequence drawn from the same generator."""
    from deeplearning4j_b200.ops import native, registry
    native.require()
    registry.load_all()
    sg = registry.get("skipgram").fn
    V = 50
    syn0, syn1, syn1n = _tables(V, D, 1)
    neg = torch.randint(0, V, (1000,), dtype=torch.int32)
    exp = torch.empty(0)
    cpu = [t.clone() for t in (syn0, syn1, syn1n)]
    gpu = [t.clone().cuda() for t in (syn0, syn1, syn1n)]
    g = torch.Generator().manual_seed(2)
    for step in range(12):
        target = torch.randint(0, V, (1,), generator=g, dtype=torch.int32)
        starter = torch.randint(0, V, (1,), generator=g, dtype=torch.int32)
        pts = torch.randperm(V - 1, generator=g)[:6].to(torch.int32).reshape(1, 6)
        pts[0, 4:] = -1
        cds = torch.randint(0, 2, (1, 6), generator=g, dtype=torch.int8)
        alpha = torch.tensor([0.05])
        rnd = torch.randint(0, 1 << 40, (1,), generator=g)
        sg(target, starter, pts, cds, cpu[0], cpu[1], cpu[2], exp, neg, alpha, rnd, nsRounds=4)
        before = native.LAUNCHES
        sg(target.cuda(), starter.cuda(), pts.cuda(), cds.cuda(), gpu[0], gpu[1], gpu[2], exp, neg.cuda(), alpha, rnd, nsRounds=4)
        assert native.LAUNCHES == before + 1                 # the whole update is one kernel
    torch.cuda.synchronize()
    for a, b in zip(cpu, gpu):
        torch.testing.assert_close(b.cpu(), a, rtol=1e-4, atol=1e-6)
    assert not torch.equal(cpu[0], syn0) and not torch.equal(cpu[1], syn1) and not torch.equal(cpu[2], syn1n)


def test_cbow_kernel_matches_the_sequential_formulation():
    from deeplearning4j_b200.ops import native, registry
    native.require()
    registry.load_all()
    cb = registry.get("cbow").fn
    V, D = 40, 64
    syn0, syn1, syn1n = _tables(V, D, 3)
    neg = torch.randint(0, V, (512,), dtype=torch.int32)
    exp = torch.empty(0)
    cpu = [t.clone() for t in (syn0, syn1, syn1n)]
    gpu = [t.clone().cuda() for t in (syn0, syn1, syn1n)]
    g = torch.Generator().manual_seed(4)
    for step in range(10):
        target = torch.randint(0, V, (1,), generator=g, dtype=torch.int32)
        ctx = torch.randperm(V, generator=g)[:6].to(torch.int32)
        ctx[5] = -1
        pts = torch.randperm(V - 1, generator=g)[:5].to(torch.int32)
        cds = torch.randint(0, 2, (5,), generator=g, dtype=torch.int8)
        alpha, rnd = torch.tensor([0.03]), torch.randint(0, 1 << 40, (1,), generator=g)
        locked = torch.empty(0)
        cb(target, target.clone(), ctx, locked, pts, cds, cpu[0], cpu[1], cpu[2], exp, neg, alpha, rnd, nsRounds=3)
        cb(target.cuda(), target.cuda(), ctx.cuda(), locked, pts.cuda(), cds.cuda(), gpu[0], gpu[1], gpu[2], exp, neg.cuda(), alpha, rnd, nsRounds=3)
    torch.cuda.synchronize()
    for a, b in zip(cpu, gpu):
        torch.testing.assert_close(b.cpu(), a, rtol=1e-4, atol=1e-6)


def test_batched_examples_update_shared_rows_without_losing_updates():
    """A batch whose examples all hit the same output row: the row must receive every example's contribution (fp32 atomics),
    up to the staleness of reading the row while others update it, which is bounded by alpha."""
    from deeplearning4j_b200.ops import native
    native.require()
    V, D, B = 64, 32, 48
    syn0 = (torch.rand(V, D) - 0.5).cuda()
    syn1n = torch.zeros(V, D).cuda()
    target = torch.arange(B, dtype=torch.int32).cuda() % V
    starter = torch.full((B,), 7, dtype=torch.int32).cuda()
    s0 = syn0.clone()
    # every negative sample is drawn from a table that only holds the positive word, so it is skipped and only the positive pair trains
    neg = torch.full((16,), 7, dtype=torch.int32).cuda()
    ok = native.w2v_batch(syn0, None, syn1n, neg, target, starter, None, None, None, torch.tensor([0.01]), torch.arange(B), 3, True)
    assert ok
    torch.cuda.synchronize()
    # row 7 of syn1neg = sum_b alpha * (1 - sigmoid(0)) * syn0[b]  (the row starts at 0 and the dot products stay tiny, so staleness is
    # second order)
    expect = 0.01 * 0.5 * s0[:B].sum(0)
    torch.testing.assert_close(syn1n[7], expect, rtol=2e-2, atol=5e-4)        # elements near zero: the staleness term dominates them
    assert float(syn1n[torch.arange(V).cuda() != 7].abs().max()) == 0.0


def test_word2vec_trains_on_the_device_through_the_batch_kernel():
    from tests.test_nlp import _cluster_score, _corpus
    from deeplearning4j_b200.nlp import CollectionSentenceIterator, DefaultTokenizerFactory, Word2Vec
    from deeplearning4j_b200.ops import native
    for kw in (dict(negativeSample=5, useHierarchicSoftmax=False), dict(negativeSample=0, useHierarchicSoftmax=True),
               dict(negativeSample=5, useHierarchicSoftmax=False, elementsLearningAlgorithm="CBOW")):
        # 64 examples per launch: the corpus has a dozen words, so larger batches make every warp race on the same few rows
        # (lock-free updates, as in the reference's host loop) and the outcome starts to depend on warp timing
        vec = (Word2Vec.Builder().minWordFrequency(1).layerSize(24).windowSize(3).epochs(16).seed(7).batchSize(64).learningRate(0.05)
               .iterate(CollectionSentenceIterator(_corpus())).tokenizerFactory(DefaultTokenizerFactory()).device("cuda").build())
        for k, v in kw.items():
            setattr(vec, k, v)
        before = native.LAUNCHES
        vec.fit()
        assert native.LAUNCHES > before, "the batch kernel did not run"
        assert _cluster_score(vec) > 0.2, (kw, _cluster_score(vec))


def test_barnes_edge_forces_kernel():
    from deeplearning4j_b200.ops import native, registry
    native.require()
    registry.load_all()
    f = registry.get("barnes_edge_forces").fn
    g = torch.Generator().manual_seed(5)
    N, D = 300, 2
    y = torch.randn(N, D, generator=g)
    deg = torch.randint(0, 9, (N,), generator=g)
    row = torch.cat([torch.zeros(1, dtype=torch.int64), deg.cumsum(0)]).to(torch.int32)
    col = torch.randint(0, N, (int(row[-1]),), generator=g, dtype=torch.int32)
    val = torch.rand(int(row[-1]), generator=g)
    ref = f(row, col, val, y)
    got = f(row.cuda(), col.cuda(), val.cuda(), y.cuda())
    torch.testing.assert_close(got.cpu(), ref, rtol=1e-4, atol=1e-6)
