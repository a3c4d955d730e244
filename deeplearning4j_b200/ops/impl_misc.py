"""Remaining op groups: TensorArray/list ops (``headers/list.h``), NLP (``headers/nlp.h``: skipgram /
cbow with hierarchical softmax + negative sampling, ``helpers/cuda/sg_cb.cu``), Barnes-Hut t-SNE
helpers (``headers/BarnesHutTsne.h``), string / compat / util / test ops, and the gradient
compression ops (``encode_threshold`` / ``decode_threshold`` / ``encode_bitmap`` / ``decode_bitmap``)."""
from __future__ import annotations

import math

import torch

from .registry import op


# ----------------------------------------------------------------------------- list (TensorArray) ops
class NDArrayList:
    def __init__(self, size=0, dtype=None):
        self.items = {}
        self.size = int(size)

    def write(self, i, v):
        self.items[int(i)] = v
        self.size = max(self.size, int(i) + 1)

    def read(self, i):
        return self.items[int(i)]

    def stack(self):
        return torch.stack([self.items[i] for i in range(self.size)])


op("create_list", differentiable=False)(lambda *a, height=0, expandable=True, **kw: NDArrayList(height))
op("write_list")(lambda lst, v, idx=None, index=0, **kw: (lst.write(int(idx) if idx is not None else index, v), lst)[1])
op("read_list")(lambda lst, idx=None, index=0, **kw: lst.read(int(idx) if idx is not None else index))
op("stack_list")(lambda lst, **kw: lst.stack())
op("size_list", differentiable=False)(lambda lst, **kw: torch.tensor(lst.size, dtype=torch.int32))
op("delete_list", differentiable=False)(lambda lst, idx=None, index=0, **kw: (lst.items.pop(int(idx) if idx is not None else index, None), lst)[1])
op("clone_list")(lambda lst, **kw: _clone_list(lst))
op("pick_list")(lambda lst, idx=None, indices=None, **kw: torch.stack([lst.read(int(i)) for i in (idx.tolist() if idx is not None else indices)]))
op("gather_list")(lambda lst, idx, **kw: torch.stack([lst.read(int(i)) for i in idx.reshape(-1).tolist()]))


def _clone_list(lst):
    n = NDArrayList(lst.size)
    n.items = dict(lst.items)
    return n


@op("unstack_list")
def unstack_list(lst, x=None, **kw):
    if x is None:
        lst, x = NDArrayList(), lst
    for i, v in enumerate(torch.unbind(x, 0)):
        lst.write(i, v)
    return lst


@op("scatter_list")
def scatter_list(lst, idx, x, **kw):
    for i, v in zip(idx.reshape(-1).tolist(), torch.unbind(x, 0)):
        lst.write(int(i), v)
    return lst


@op("split_list")
def split_list(lst, x, sizes, **kw):
    off = 0
    for i, s in enumerate(sizes.reshape(-1).tolist()):
        lst.write(i, x[off:off + int(s)])
        off += int(s)
    return lst


# ----------------------------------------------------------------------------- word2vec
_MAX_EXP = 6.0      # HS_MAX_EXP of helpers/cuda/sg_cb.cu


def _native_w2v(syn0, syn1, syn1neg, negTable, target, ngStarter, indices, codes, context, alpha, randomValue, nsRounds, trainWords=True):
    """The whole batch in one kernel launch when the tables are fp32 CUDA tensors."""
    if not (isinstance(syn0, torch.Tensor) and syn0.is_cuda and syn0.dtype == torch.float32):
        return False
    from . import native
    if not native.available():
        return False
    s1 = syn1 if syn1 is not None and syn1.numel() else None
    s1n = syn1neg if syn1neg is not None and syn1neg.numel() else None
    pts = indices if indices is not None and indices.numel() and s1 is not None else None
    ng = ngStarter if ngStarter is not None and ngStarter.numel() else None
    return native.w2v_batch(syn0, s1, s1n, negTable, target, ng, pts, codes if pts is not None else None, context, alpha, randomValue,
                            nsRounds if ng is not None else 0, trainWords)


def _sg_rows(syn0, syn1, syn1neg, expTable, target, codes, points, ngStarter, negTable, alpha, nsRounds, nextRandom, vec=None, train_vec=True):
    """One skip-gram style update of row ``target`` of syn0 (or of ``vec`` in inference mode).  Output rows are visited one after
    the other, each seeing the updates of the ones before it, as ``helpers/cuda/sg_cb.cu`` does (hSoftmax_ / nSampling_ per row)."""
    l1 = (vec if vec is not None else syn0[target]).clone()
    neu1e = torch.zeros_like(l1)

    def row_step(table, r, code, hierarchic):
        row = table[r]
        dot = float(row @ l1)
        if hierarchic:
            if dot < -_MAX_EXP or dot >= _MAX_EXP:          # saturated node: skipped
                return
            g = (1.0 - code - 1.0 / (1.0 + math.exp(-dot))) * alpha
        elif dot > _MAX_EXP:
            g = (code - 1.0) * alpha
        elif dot < -_MAX_EXP:
            g = code * alpha
        else:
            g = (code - 1.0 / (1.0 + math.exp(-dot))) * alpha
        neu1e.add_(row, alpha=g)
        table[r] = row + g * l1

    if points is not None and len(points) and syn1 is not None:
        for p_, c_ in zip(points.tolist(), codes.tolist()):
            row_step(syn1, int(p_), float(c_), True)
    if nsRounds > 0 and syn1neg is not None and int(ngStarter) >= 0:
        r = int(nextRandom) & 0xFFFFFFFFFFFFFFFF
        nt = negTable
        row_step(syn1neg, int(ngStarter), 1.0, False)
        for _ in range(int(nsRounds)):
            r = (r * 25214903917 + 11) & 0xFFFFFFFFFFFFFFFF
            t = int(nt[(r >> 16) % nt.numel()]) if nt is not None and nt.numel() else (r >> 16) % syn1neg.shape[0]
            if t == int(ngStarter):
                continue
            row_step(syn1neg, t, 0.0, False)
    if train_vec:
        if vec is not None:
            vec += neu1e
        else:
            syn0[target] += neu1e
    return neu1e


@op("skipgram", differentiable=False, n_out=-1)
def skipgram(target, ngStarter, indices, codes, syn0, syn1, syn1neg, expTable, negTable, alpha, randomValue, inferenceVector=None,
             nsRounds=0, isInference=False, isPreciseMode=False, numWorkers=1, **kw):
    if not isInference and inferenceVector is None and _native_w2v(syn0, syn1, syn1neg, negTable, target, ngStarter, indices, codes, None,
                                                                     alpha, randomValue, nsRounds):
        return (syn0, syn1, syn1neg)
    tg = target.reshape(-1).tolist()
    al = alpha.reshape(-1).tolist()
    rv = randomValue.reshape(-1).tolist()
    ng = ngStarter.reshape(-1).tolist() if ngStarter is not None and ngStarter.numel() else [-1] * len(tg)
    idx2 = indices.reshape(len(tg), -1) if indices is not None and indices.numel() else None
    cod2 = codes.reshape(len(tg), -1) if codes is not None and codes.numel() else None
    for i, t in enumerate(tg):
        pts = cds = None
        if idx2 is not None:
            valid = idx2[i] >= 0
            pts, cds = idx2[i][valid].long(), cod2[i][valid]
        _sg_rows(syn0, syn1 if syn1 is not None and syn1.numel() else None, syn1neg if syn1neg is not None and syn1neg.numel() else None,
                 expTable, int(t), cds, pts, ng[i], negTable, al[i % len(al)], nsRounds if ng[i] >= 0 else 0, rv[i % len(rv)],
                 vec=inferenceVector if isInference else None)
    return (syn0, syn1, syn1neg)


op("skipgram_inference", differentiable=False, n_out=-1)(lambda *a, **kw: skipgram(*a, isInference=True, **kw))


@op("cbow", differentiable=False, n_out=-1)
def cbow(target, ngStarter, context, lockedWords, indices, codes, syn0, syn1, syn1neg, expTable, negTable, alpha, randomValue,
         numLabels=None, inferenceVector=None, nsRounds=0, trainWords=True, isInference=False, **kw):
    if not isInference and inferenceVector is None and target.numel() >= 1 and context.numel() % target.numel() == 0 \
            and _native_w2v(syn0, syn1, syn1neg, negTable, target, ngStarter, indices, codes, context.reshape(target.numel(), -1), alpha,
                            randomValue, nsRounds, trainWords):
        return (syn0, syn1, syn1neg)
    ctx = context.reshape(-1)
    ctx = ctx[ctx >= 0].long()
    if ctx.numel() == 0 and inferenceVector is None:
        return (syn0, syn1, syn1neg)
    neu1 = syn0[ctx].sum(0) if ctx.numel() else torch.zeros(syn0.shape[1], dtype=syn0.dtype, device=syn0.device)
    cnt = ctx.numel()
    if inferenceVector is not None:
        neu1 = neu1 + inferenceVector
        cnt += 1
    neu1 = neu1 / max(cnt, 1)
    pts = cds = None
    if indices is not None and indices.numel():
        valid = indices.reshape(-1) >= 0
        pts, cds = indices.reshape(-1)[valid].long(), codes.reshape(-1)[valid]
    ng = int(ngStarter.reshape(-1)[0]) if ngStarter is not None and ngStarter.numel() else -1
    neu1e = _sg_rows(syn0, syn1 if syn1 is not None and syn1.numel() else None, syn1neg if syn1neg is not None and syn1neg.numel() else None,
                     expTable, int(target.reshape(-1)[0]), cds, pts, ng, negTable, float(alpha.reshape(-1)[0]),
                     nsRounds if ng >= 0 else 0, int(randomValue.reshape(-1)[0]), vec=neu1, train_vec=False)
    if isInference and inferenceVector is not None:
        inferenceVector += neu1e
    elif trainWords and ctx.numel():
        syn0.index_add_(0, ctx, neu1e.unsqueeze(0).expand(ctx.numel(), -1))
    return (syn0, syn1, syn1neg)


op("cbow_inference", differentiable=False, n_out=-1)(lambda *a, **kw: cbow(*a, isInference=True, **kw))


# ----------------------------------------------------------------------------- Barnes-Hut t-SNE helpers
@op("barnes_gains")
def barnes_gains(gains, gradX, epsilon, **kw):
    same = torch.sign(gradX) == torch.sign(epsilon)
    return torch.where(same, gains * 0.8, gains + 0.2).clamp_min(0.01)


@op("barnes_edge_forces")
def barnes_edge_forces(rowP, colP, valP, dataP, N=None, **kw):
    n = int(N) if N is not None else dataP.shape[0]
    if dataP.is_cuda and dataP.dtype == torch.float32 and n == dataP.shape[0]:
        from . import native
        r = native.barnes_edge_forces(rowP, colP, valP, dataP) if native.available() else None
        if r is not None:
            return r
    out = torch.zeros_like(dataP)
    rp = rowP.long().tolist()
    for i in range(n):
        js = colP[rp[i]:rp[i + 1]].long()
        if js.numel() == 0:
            continue
        d = dataP[i].unsqueeze(0) - dataP[js]
        w = valP[rp[i]:rp[i + 1]] / (1.0 + (d * d).sum(1))
        out[i] = (w.unsqueeze(1) * d).sum(0)
    return out


@op("barnes_symmetrized", n_out=3, differentiable=False)
def barnes_symmetrized(rowP, colP, valP, N=None, **kw):
    n = int(N) if N is not None else rowP.numel() - 1
    rp = rowP.long()
    rows = torch.repeat_interleave(torch.arange(n, device=rowP.device), rp[1:] - rp[:-1])
    P = torch.sparse_coo_tensor(torch.stack([rows, colP.long()]), valP.float(), (n, n)).coalesce()
    S = ((P + P.t()) * 0.5).coalesce()
    r, c = S.indices()
    cnt = torch.bincount(r, minlength=n)
    return torch.cat([torch.zeros(1, dtype=torch.int64, device=r.device), cnt.cumsum(0)]).to(rowP.dtype), c.to(colP.dtype), S.values().to(valP.dtype)


@op("cell_contains", differentiable=False)
def cell_contains(corner, width, point, dimension=None, **kw):
    return ((corner - width <= point) & (point <= corner + width)).all()


# ----------------------------------------------------------------------------- strings / compat / util / tests
op("split_string", differentiable=False)(lambda s, delim=" ", **kw: (s if isinstance(s, str) else str(s)).split(delim if isinstance(delim, str) else str(delim)))


@op("compat_string_split", n_out=2, differentiable=False)
def compat_string_split(strings, delim=" ", **kw):
    idx, vals = [], []
    for i, s in enumerate(strings):
        for j, tok in enumerate(str(s).split(delim if isinstance(delim, str) else str(delim))):
            idx.append([i, j])
            vals.append(tok)
    return torch.tensor(idx, dtype=torch.int64), vals


@op("compat_sparse_to_dense")
def compat_sparse_to_dense(indices, shape, values, default=None, **kw):
    s = [int(v) for v in shape.reshape(-1).tolist()]
    out = torch.full(s, float(default) if default is not None else 0.0, dtype=values.dtype, device=values.device)
    idx = indices.long().reshape(-1, len(s))
    out[tuple(idx[:, i] for i in range(len(s)))] = values
    return out


@op("print_variable", differentiable=False)
def print_variable(x, message="", printSpecial=False, **kw):
    print(message, x)
    return x


op("print_affinity", differentiable=False)(lambda x, **kw: (print(f"device: {x.device}"), x)[1])
op("Assert", differentiable=False)(lambda cond, *data, **kw: _assert(cond))


def _assert(cond):
    if not bool(cond.all()):
        raise AssertionError("Assert op failed")
    return cond


op("test_output_reshape")(lambda x, **kw: x.reshape(-1))
op("test_scalar")(lambda x, **kw: x.reshape(-1)[:1] * 2)
op("testreduction")(lambda x, **kw: x.sum())
op("testop2i2o", n_out=2)(lambda x, y, **kw: (x + 1, y + 2))
op("testcustom")(lambda x, **kw: x)


# ----------------------------------------------------------------------------- gradient compression as ops
@op("encode_threshold", n_out=2, differentiable=False)
def encode_threshold(x, threshold=1e-3, boundary=None, **kw):
    from ..parallel import codec
    r = x.clone().reshape(-1).float()
    msg = codec.threshold_encode(r, float(threshold), None if boundary is None else int(boundary))
    return r.reshape(x.shape).to(x.dtype), msg


@op("decode_threshold", differentiable=False)
def decode_threshold(x, encoded, **kw):
    from ..parallel import codec
    out = x.clone().float()
    codec.threshold_decode(encoded, out)
    return out.to(x.dtype)


@op("encode_bitmap", n_out=3, differentiable=False)
def encode_bitmap(x, threshold=1e-3, **kw):
    from ..parallel import codec
    r = x.clone().reshape(-1).float()
    msg = codec.bitmap_encode(r, float(threshold))
    return r.reshape(x.shape).to(x.dtype), msg, msg[0:1].clone()


@op("decode_bitmap", differentiable=False)
def decode_bitmap(x, encoded, **kw):
    from ..parallel import codec
    out = x.clone().float()
    codec.bitmap_decode(encoded, out)
    return out.to(x.dtype)


# ----------------------------------------------------------------------------- TensorFlow-style TensorArray ops
# Graphs imported from TensorFlow (and the reference's .fb files made from them) thread a scalar "flow" value through the
# TensorArray ops to order them: write / scatter / split return the flow, read / gather / size / concat take it as their last input
# (libnd4j/include/ops/declarable/generic/list/*.cpp under their tensorarray*v3 synonyms).
def _flow():
    return torch.zeros((), dtype=torch.float32)


@op("tf_list_create", n_out=2, differentiable=False)
def tf_list_create(size=None, **kw):
    n = int(torch.as_tensor(size).reshape(-1)[0]) if size is not None else 0
    return NDArrayList(max(n, 0)), _flow()


@op("tf_list_write", differentiable=False)
def tf_list_write(lst, idx, v, flow=None, **kw):
    lst.write(int(torch.as_tensor(idx).reshape(-1)[0]), v)
    return _flow()


@op("tf_list_read")
def tf_list_read(lst, idx, flow=None, **kw):
    return lst.read(int(torch.as_tensor(idx).reshape(-1)[0]))


@op("tf_list_gather")
def tf_list_gather(lst, idx, flow=None, **kw):
    return torch.stack([lst.read(int(i)) for i in torch.as_tensor(idx).reshape(-1).tolist()])


@op("tf_list_scatter", differentiable=False)
def tf_list_scatter(lst, idx, x, flow=None, **kw):
    for k, i in enumerate(torch.as_tensor(idx).reshape(-1).tolist()):
        lst.write(int(i), x[k])
    return _flow()


@op("tf_list_split", differentiable=False)
def tf_list_split(lst, x, sizes, flow=None, **kw):
    pos = 0
    for k, n in enumerate(torch.as_tensor(sizes).reshape(-1).tolist()):
        lst.write(k, x[pos:pos + int(n)])
        pos += int(n)
    return _flow()


@op("tf_list_size", differentiable=False)
def tf_list_size(lst, flow=None, **kw):
    return torch.tensor(lst.size, dtype=torch.int64)


@op("tf_list_concat")
def tf_list_concat(lst, flow=None, **kw):
    return torch.cat([lst.read(i) for i in range(lst.size)], 0)
