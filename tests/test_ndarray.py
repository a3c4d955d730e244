"""INDArray / Nd4j factory behaviour against numpy (ordering, views, indexing, in-place ops, reductions, linear
algebra, binary / npy / text IO).  Mirrors the intent of nd4j's Nd4jTestsC / NDArrayTestsFortran."""
import io

import numpy as np
import pytest
import torch

from deeplearning4j_b200 import DataType, INDArray, NDArrayIndex, Nd4j, Transforms


def _np(a):
    return a.numpy() if isinstance(a, INDArray) else np.asarray(a)


def test_create_shapes_orders_and_dtypes():
    a = Nd4j.create([[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]])
    assert a.shape() == (2, 3) and a.rank() == 2 and a.length() == 6
    assert a.rows() == 2 and a.columns() == 3 and a.isMatrix() and not a.isVector()
    assert a.ordering() == "c"
    f = Nd4j.create([1.0, 2.0, 3.0, 4.0, 5.0, 6.0], shape=(2, 3), order="f")
    assert f.ordering() == "f"
    # fortran order fills columns first
    np.testing.assert_array_equal(_np(f), np.array([[1, 3, 5], [2, 4, 6]], dtype=np.float32))
    z = Nd4j.zeros(3, 4, dtype=DataType.DOUBLE)
    assert z.dataType() == DataType.DOUBLE and float(z.sumNumber()) == 0.0
    o = Nd4j.ones(5)
    assert o.isVector() and float(o.sumNumber()) == 5.0
    s = Nd4j.scalar(3.5)
    assert s.isScalar() and s.getDouble() == 3.5
    e = Nd4j.eye(3)
    np.testing.assert_array_equal(_np(e), np.eye(3, dtype=np.float32))
    v = Nd4j.valueArrayOf((2, 2), 7.0)
    assert float(v.meanNumber()) == 7.0
    li = Nd4j.linspace(1, 10, 10)
    np.testing.assert_allclose(_np(li), np.linspace(1, 10, 10), rtol=1e-6)
    assert Nd4j.arange(5).toIntVector() == [0, 1, 2, 3, 4]


def test_cast_and_dup_independence():
    a = Nd4j.create([[1.5, 2.5], [3.5, 4.5]])
    i = a.castTo(DataType.INT)
    assert i.dataType() == DataType.INT and i.toIntVector() == [1, 2, 3, 4]
    d = a.dup()
    d.addi(1.0)
    assert a.getDouble(0, 0) == 1.5 and d.getDouble(0, 0) == 2.5
    h = a.castTo(DataType.BFLOAT16)
    assert h.dataType() == DataType.BFLOAT16


def test_views_share_memory_and_assign():
    a = Nd4j.zeros(4, 5)
    row = a.getRow(1)
    row.assign(3.0)
    assert float(a.sumNumber()) == 15.0
    col = a.getColumn(2)
    col.addi(1.0)
    assert a.getDouble(0, 2) == 1.0 and a.getDouble(1, 2) == 4.0
    sub = a.get(NDArrayIndex.interval(0, 2), NDArrayIndex.all())
    assert sub.shape() == (2, 5)
    sub.muli(2.0)
    assert a.getDouble(1, 0) == 6.0
    p = a.get(NDArrayIndex.point(1), NDArrayIndex.interval(1, 3))
    np.testing.assert_array_equal(_np(p).ravel(), np.array([6.0, 8.0], dtype=np.float32))
    a.put((NDArrayIndex.point(3), NDArrayIndex.all()), Nd4j.ones(5))
    assert float(a.getRow(3).sumNumber()) == 5.0
    a.putScalar((0, 0), 9.0)
    assert a.getDouble(0, 0) == 9.0


def test_reshape_permute_transpose_match_numpy():
    x = np.arange(24, dtype=np.float32).reshape(2, 3, 4)
    a = Nd4j.create(x)
    np.testing.assert_array_equal(_np(a.reshape(6, 4)), x.reshape(6, 4))
    np.testing.assert_array_equal(_np(a.permute(2, 0, 1)), x.transpose(2, 0, 1))
    np.testing.assert_array_equal(_np(a.swapAxes(0, 2)), x.swapaxes(0, 2))
    m = Nd4j.create(x.reshape(6, 4))
    np.testing.assert_array_equal(_np(m.transpose()), x.reshape(6, 4).T)
    np.testing.assert_array_equal(_np(a.ravel()), x.ravel())
    tad = a.tensorAlongDimension(1, 1, 2)
    np.testing.assert_array_equal(_np(tad), x[1])
    assert a.tensorsAlongDimension(1, 2) == 2


def test_arithmetic_broadcast_and_inplace():
    x = np.arange(6, dtype=np.float32).reshape(2, 3) + 1
    a = Nd4j.create(x)
    np.testing.assert_allclose(_np(a.add(1.0)), x + 1)
    np.testing.assert_allclose(_np(a.rsub(10.0)), 10 - x)
    np.testing.assert_allclose(_np(a.rdiv(6.0)), 6 / x)
    np.testing.assert_allclose(_np(a.mul(a)), x * x)
    np.testing.assert_allclose(_np(a.neg()), -x)
    r = Nd4j.create([10.0, 20.0, 30.0])
    c = Nd4j.create([[100.0], [200.0]])
    np.testing.assert_allclose(_np(a.addRowVector(r)), x + np.array([10, 20, 30]))
    np.testing.assert_allclose(_np(a.mulColumnVector(c)), x * np.array([[100], [200]]))
    b = a.dup()
    b.subiRowVector(r).divi(2.0)
    np.testing.assert_allclose(_np(b), (x - np.array([10, 20, 30])) / 2)
    assert a.gt(3.0).castTo(DataType.INT).sumNumber() == 3
    assert bool(a.eq(a).all()) and not bool(a.neq(a).any())


def test_reductions_match_numpy():
    rng = np.random.default_rng(0)
    x = rng.normal(size=(4, 5, 6)).astype(np.float32)
    a = Nd4j.create(x)
    np.testing.assert_allclose(_np(a.sum(1)), x.sum(1), rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(_np(a.mean(0, 2)), x.mean((0, 2)), rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(_np(a.max(2)), x.max(2))
    np.testing.assert_allclose(_np(a.min(0)), x.min(0))
    np.testing.assert_allclose(_np(a.std(1)), x.std(1, ddof=1), rtol=1e-4)          # bias-corrected by default
    np.testing.assert_allclose(_np(a.var(1)), x.var(1, ddof=1), rtol=1e-4)
    np.testing.assert_allclose(_np(a.norm1(2)), np.abs(x).sum(2), rtol=1e-5)
    np.testing.assert_allclose(_np(a.norm2(2)), np.sqrt((x * x).sum(2)), rtol=1e-5)
    np.testing.assert_allclose(_np(a.normmax(2)), np.abs(x).max(2))
    np.testing.assert_allclose(_np(a.prod(0)), x.prod(0), rtol=1e-4)
    np.testing.assert_array_equal(_np(a.argMax(2)), x.argmax(2))
    np.testing.assert_allclose(_np(a.cumsum(1)), x.cumsum(1), rtol=1e-5, atol=1e-5)
    assert abs(float(a.sumNumber()) - float(x.sum())) < 1e-3
    assert abs(float(a.norm2Number()) - float(np.sqrt((x * x).sum()))) < 1e-3


def test_linear_algebra():
    rng = np.random.default_rng(1)
    x, y = rng.normal(size=(3, 4)).astype(np.float32), rng.normal(size=(4, 5)).astype(np.float32)
    a, b = Nd4j.create(x), Nd4j.create(y)
    np.testing.assert_allclose(_np(a.mmul(b)), x @ y, rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(_np(Nd4j.gemm(a, a, False, True)), x @ x.T, rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(_np(Nd4j.matmul(a, b, transposeResult=True)), (x @ y).T, rtol=1e-5, atol=1e-5)
    t = Nd4j.tensorMmul(Nd4j.create(rng.normal(size=(2, 3, 4)).astype(np.float32)), b, [[2], [0]])
    assert t.shape() == (2, 3, 5)
    v = Nd4j.create([1.0, 2.0, 3.0])
    assert float(v.dot(v)) == 14.0
    assert abs(Transforms.cosineSim(v, v) - 1.0) < 1e-6
    assert abs(Transforms.euclideanDistance(v, Nd4j.zeros(3)) - np.sqrt(14.0)) < 1e-5
    assert abs(Transforms.manhattanDistance(v, Nd4j.zeros(3)) - 6.0) < 1e-6


def test_concat_stack_tile_sort_where():
    a, b = Nd4j.ones(2, 3), Nd4j.zeros(2, 3)
    assert Nd4j.concat(0, a, b).shape() == (4, 3)
    assert Nd4j.hstack(a, b).shape() == (2, 6)
    assert Nd4j.vstack(a, b).shape() == (4, 3)
    assert Nd4j.stack(0, a, b).shape() == (2, 2, 3)
    assert Nd4j.pile(a, b).shape() == (2, 2, 3)
    assert Nd4j.tile(a, 2, 2).shape() == (4, 6)
    fl = Nd4j.toFlattened(a, b)
    assert fl.length() == 12 and float(fl.sumNumber()) == 6.0
    s = Nd4j.sort(Nd4j.create([3.0, 1.0, 2.0]), 0, True)
    assert s.toDoubleVector() == [1.0, 2.0, 3.0]
    w = Nd4j.where(Nd4j.create([1.0, 0.0]).gt(0.5), Nd4j.create([5.0, 5.0]), Nd4j.create([7.0, 7.0]))
    assert w.toDoubleVector() == [5.0, 7.0]


def test_transforms_elementwise():
    x = np.linspace(-2, 2, 9).astype(np.float32)
    a = Nd4j.create(x)
    np.testing.assert_allclose(_np(Transforms.sigmoid(a)), 1 / (1 + np.exp(-x)), rtol=1e-5)
    np.testing.assert_allclose(_np(Transforms.tanh(a)), np.tanh(x), rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(_np(Transforms.relu(a)), np.maximum(x, 0))
    np.testing.assert_allclose(_np(Transforms.exp(a)), np.exp(x), rtol=1e-5)
    np.testing.assert_allclose(_np(Transforms.abs(a)), np.abs(x))
    np.testing.assert_allclose(_np(Transforms.pow(a, 2)), x ** 2, rtol=1e-6)
    sm = _np(Transforms.softmax(Nd4j.create(x.reshape(1, -1))))
    np.testing.assert_allclose(sm.sum(), 1.0, rtol=1e-6)
    u = Transforms.unitVec(Nd4j.create([3.0, 4.0]))
    np.testing.assert_allclose(_np(u), [0.6, 0.8], rtol=1e-6)
    # dup=False works in place
    b = Nd4j.create(x.copy())
    Transforms.relu(b, False)
    assert float(b.minNumber()) == 0.0


def test_binary_npy_and_text_io(tmp_path):
    rng = np.random.default_rng(2)
    x = rng.normal(size=(3, 4)).astype(np.float32)
    a = Nd4j.create(x)
    buf = io.BytesIO()
    Nd4j.write(a, buf)
    buf.seek(0)
    back = Nd4j.read(buf)
    assert back.equals(a) and back.dataType() == a.dataType() and back.ordering() == a.ordering()
    f = Nd4j.create(x.T.copy().ravel().tolist(), shape=(3, 4), order="f")
    raw = Nd4j.toByteArray(f)
    g = Nd4j.fromByteArray(raw)
    assert g.ordering() == "f" and g.equals(f)
    p = str(tmp_path / "a.bin")
    Nd4j.saveBinary(a, p)
    assert Nd4j.readBinary(p).equals(a)
    npy = str(tmp_path / "a.npy")
    Nd4j.writeAsNumpy(a, npy)
    np.testing.assert_array_equal(np.load(npy), x)
    assert Nd4j.createFromNpyFile(npy).equals(a)
    assert Nd4j.createNpyFromByteArray(Nd4j.toNpyByteArray(a)).equals(a)
    txt = str(tmp_path / "a.txt")
    Nd4j.writeTxt(a, txt)
    assert Nd4j.readTxt(txt).equalsWithEps(a, 1e-5)


def test_random_is_seeded():
    Nd4j.getRandom().setSeed(123)
    a = Nd4j.rand(3, 3)
    Nd4j.getRandom().setSeed(123)
    b = Nd4j.rand(3, 3)
    assert a.equals(b)
    n = Nd4j.randn(2000, seed=7)
    assert abs(float(n.meanNumber())) < 0.1 and abs(float(n.stdNumber()) - 1.0) < 0.1
    bern = Nd4j.randomBernoulli(0.3, 4000)
    assert abs(float(bern.meanNumber()) - 0.3) < 0.05


def test_equality_and_distance_helpers():
    a = Nd4j.create([1.0, 2.0, 3.0])
    b = Nd4j.create([1.0, 2.0, 3.0 + 1e-7])
    assert a.equalsWithEps(b, 1e-5) and a.equalShapes(b)
    assert not a.equalsWithEps(Nd4j.create([1.0, 2.0, 4.0]), 1e-5)
    assert abs(a.distance2(Nd4j.zeros(3)) - np.sqrt(14.0)) < 1e-5
    assert abs(a.distance1(Nd4j.zeros(3)) - 6.0) < 1e-6
    assert abs(a.squaredDistance(Nd4j.zeros(3)) - 14.0) < 1e-5


def test_counter_based_random_generator_matches_scalar_arithmetic():
    from deeplearning4j_b200.nd.rng import RandomGenerator
    root, node = 119, 5
    g = RandomGenerator(root, node)
    M64, M32 = (1 << 64) - 1, (1 << 32) - 1

    def x32(index):                                   # the stream definition written out with Python integers
        s0 = root | (((index + 2) * (node + 24243287)) & M64)
        s1 = node ^ (((index + 2) * (s0 + 723829)) & M64)
        half = (s1 ^ s0) & M32
        x = (half * 0x9E3779BB) & M32
        x = ((x << 5) | (x >> 27)) & M32
        return (x * 5) & M32
    idx = np.array([0, 1, 2, 1000, 123456789], dtype=np.uint64)
    assert g.xoroshiro32(idx).tolist() == [x32(int(i)) for i in idx]
    f = g.relativeFloat(idx)
    want = [np.frombuffer(np.uint32(0x3F800000 | (x32(int(i)) >> 9)).tobytes(), dtype=np.float32)[0] - np.float32(1.0) for i in idx]
    np.testing.assert_array_equal(f, np.array(want, dtype=np.float32))
    u = g.uniform((20000,), 2.0, 4.0)
    assert float(u.min()) >= 2.0 and float(u.max()) < 4.0 and abs(float(u.mean()) - 3.0) < 0.05
    state_after = g.nodeState()
    g2 = RandomGenerator(root, node)
    g2.uniform((20000,), 2.0, 4.0)
    assert g2.nodeState() == state_after != node                       # consuming values advances the node state deterministically
    d = g.relativeDouble(np.arange(1000, dtype=np.uint64))
    assert d.min() >= 0.0 and d.max() < 1.0 and 0.4 < d.mean() < 0.6


def test_counter_based_random_generator_golden_values():
    """Literal values obtained by evaluating the stream definition of ``libnd4j/include/graph/RandomGenerator.h`` (``xoroshiro32``
    :374-385, ``xoroshiro64`` :387-393, ``relativeT<float>`` / ``<double>`` :141-156, ``rewindH`` :395-404) with plain C integer
    arithmetic (uint64 / uint32 wrap-around, the low 32 bits of ``s1 ^ s0`` taken as ``int``), independently of this package."""
    from deeplearning4j_b200.nd.rng import RandomGenerator
    g = RandomGenerator(119, 5)
    idx = np.array([0, 1, 2, 1000, 123456789], dtype=np.uint64)
    assert g.xoroshiro32(idx).tolist() == [3752294361, 3177379693, 1663668732, 1377381342, 3039950299]
    assert g.xoroshiro64(idx).tolist() == [16115981569212512217, 13646741872161814489, 7145402799070083033, 5915807821762885593,
                                           13056487119422715865]
    np.testing.assert_array_equal(g.relativeFloat(idx), np.array([0.873649001, 0.739791274, 0.387352943, 0.320696473, 0.707793474],
                                                                 dtype=np.float32))
    np.testing.assert_array_equal(g.relativeDouble(idx), np.array([0.87364911145382762, 0.73979135925733686, 0.38735306190178931,
                                                                   0.32069658461810291, 0.70779358499535561]))
    g.rewindH(20000)
    assert g.nodeState() == 175925260843722
    g.rewindH(7)
    assert g.nodeState() == -6099745996984563767
    # default node seed (a zero node seed selects 1298567341)
    assert RandomGenerator(0x123456789ABCDEF, 0).xoroshiro32(np.arange(3)).tolist() == [3946914084, 4080556201, 4230060595]


def test_conditions_boolean_indexing_and_the_rest_of_the_indarray_surface():
    from deeplearning4j_b200.nd.conditions import And, BooleanIndexing, Conditions, Not, Or
    a = Nd4j.create([[1.0, -2.0, 3.0], [-4.0, 5.0, 6.0]])
    assert a.cond(Conditions.greaterThan(0)).t.tolist() == [[1, 0, 1], [0, 1, 1]]
    assert a.scan(Conditions.absGreaterThan(3.5)) == 3
    assert a.getWhere(0.0, Conditions.lessThan(0)).t.tolist() == [-2.0, -4.0]
    assert a.putWhere(0.0, 9.0, Conditions.lessThan(0)).t.tolist() == [[1, 9, 3], [9, 5, 6]]
    assert a.putWhereWithMask(Nd4j.create([[1.0, 0, 0], [0, 0, 1.0]]), 7.0).t.tolist() == [[7, -2, 3], [-4, 5, 7]]
    b = a.dup()
    BooleanIndexing.replaceWhere(b, 0.0, And(Conditions.greaterThan(0), Not(Conditions.greaterThan(4))))
    assert b.t.tolist() == [[0, -2, 0], [-4, 5, 6]]
    assert BooleanIndexing.or_(a, Conditions.greaterThan(5)) and not BooleanIndexing.and_(a, Conditions.greaterThan(0))
    assert BooleanIndexing.firstIndex(a, Conditions.lessThan(0)).t.item() == 1
    assert BooleanIndexing.lastIndex(a, Or(Conditions.lessThan(-3), Conditions.equals(1.0))).t.item() == 3
    assert BooleanIndexing.firstIndex(a, Conditions.greaterThan(2), 1).t.tolist() == [2, 1]
    assert Conditions.fromInt(4, 1.0).name == "lessThanOrEqual" and Conditions.epsEquals(1.0).condtionNum() == 0
    c = a.dup().assignIf(Nd4j.create([[10.0, 0, 0], [0, 20.0, 0]]), Conditions.greaterThan(5))
    assert c.t.tolist() == [[10, -2, 3], [-4, 20, 6]]
    # reverse row / column vector arithmetic
    r, col = Nd4j.create([1.0, 2.0, 3.0]), Nd4j.create([10.0, 20.0])
    assert a.rsubRowVector(r).t.tolist() == [[0, 4, 0], [5, -3, -3]]
    assert torch.allclose(a.rdivColumnVector(col).t, torch.tensor([[10, -5, 10 / 3], [-5, 4, 20 / 6]]))
    assert a.dup().putiRowVector(r).t.tolist() == [[1, 2, 3], [1, 2, 3]]
    assert a.dup().rsubiColumnVector(col).t.tolist() == [[9, 12, 7], [24, 15, 14]]
    # percentile / median as the reference defines them (position q / 100 * (n + 1) on the sorted copy)
    v = Nd4j.create([3.0, 1.0, 4.0, 1.0, 5.0, 9.0, 2.0, 6.0])
    assert v.medianNumber() == 3.5 and v.percentileNumber(100) == 9.0 and v.percentileNumber(0) == 1.0
    assert abs(v.percentileNumber(25) - 1.25) < 1e-12
    assert a.median(1).t.tolist() == [1.0, 5.0]
    assert a.amaxNumber() == 6.0 and a.aminNumber() == 1.0 and abs(a.ameanNumber() - 3.5) < 1e-12
    p = Nd4j.create([0.5, 0.25, 0.25])
    assert abs(p.shannonEntropyNumber() - 1.5) < 1e-12 and abs(p.entropyNumber() - 1.5 * np.log(2)) < 1e-12
    # shapes
    m = Nd4j.create(np.arange(24.0).reshape(2, 3, 4))
    assert m.dup().permutei(2, 0, 1).shape() == (4, 2, 3) and Nd4j.create(np.eye(3)).isSquare()
    assert m.dimShuffle([1, "x", 0, 2]).shape() == (3, 1, 2, 4)
    assert m.vectorsAlongDimension(2) == 6 and len(m.sliceVectors()) == 6 and m.slices() == 2
    assert Nd4j.create(np.zeros((1, 1, 5, 1))).getLeadingOnes() == 2 and Nd4j.create(np.zeros((1, 1, 5, 1))).getTrailingOnes() == 1
    info = m.shapeInfoJava()
    assert info[0] == 3 and info[1:4] == [2, 3, 4] and info[4:7] == [12, 4, 1] and info[-1] == ord("c")
    assert "Rank: 3" in m.shapeInfoToString() and m.getNumber(1, 2, 3) == 23.0 and m.getDoubleUnsafe(5) == 5.0
    assert m.toIntMatrix()[1][0] == 12 and Nd4j.create([1.0, 2.0]).isVectorOrScalar()
    fa = m.toFlatArray()
    from deeplearning4j_b200.samediff.serde.flatgraph import from_flat_array
    assert torch.equal(from_flat_array(fa).double(), m.t.double())


def test_nd4j_factory_reductions_shapes_and_eager_namespaces():
    a = Nd4j.create([[1.0, 2, 3], [4, 5, 6]])
    assert Nd4j.sum(a, 0).t.tolist() == [5, 7, 9] and Nd4j.max(a, 1).t.tolist() == [3, 6] and float(Nd4j.prod(a).t) == 720
    assert abs(float(Nd4j.norm2(a).t) - np.sqrt(91.0)) < 1e-5 and float(Nd4j.norm1(a).t) == 21 and float(Nd4j.normmax(a).t) == 6
    assert Nd4j.append(a, 2, 9.0, 1).t.tolist() == [[1, 2, 3, 9, 9], [4, 5, 6, 9, 9]]
    assert Nd4j.prepend(a, 1, 0.0, 0).t.tolist() == [[0, 0, 0], [1, 2, 3], [4, 5, 6]]
    assert Nd4j.appendBias(Nd4j.create([1.0, 2.0]), Nd4j.create([3.0])).t.reshape(-1).tolist() == [1, 2, 3, 1]
    assert Nd4j.pad(a, [[1, 1], [0, 2]]).shape() == (4, 5) and Nd4j.pullRows(a, 1, [1, 0]).t.tolist() == [[4, 5, 6], [1, 2, 3]]
    assert Nd4j.sortRows(Nd4j.create([[3.0, 1], [1, 2], [2, 0]]), 0).t.tolist() == [[1, 2], [2, 0], [3, 1]]
    assert Nd4j.sortColumns(Nd4j.create([[3.0, 1, 2], [0, 1, 2]]), 0).t.tolist() == [[1, 2, 3], [1, 2, 0]]
    assert Nd4j.getStrides([2, 3, 4]) == [12, 4, 1] and Nd4j.getStrides([2, 3, 4], "f") == [1, 2, 6]
    assert Nd4j.reverse(Nd4j.create([1.0, 2, 3])).t.tolist() == [3, 2, 1] and Nd4j.rot90(a).shape() == (3, 2)
    assert Nd4j.rollAxis(Nd4j.create(np.zeros((2, 3, 4))), 2).shape() == (4, 2, 3)
    assert Nd4j.stripOnes(Nd4j.create(np.zeros((1, 3, 1, 2)))).shape() == (3, 2) and Nd4j.expandDims(a, 0).shape() == (1, 2, 3)
    assert Nd4j.tri(3).t.tolist() == [[1, 0, 0], [1, 1, 0], [1, 1, 1]] and Nd4j.triu(a, 1).t.tolist() == [[0, 2, 3], [0, 0, 6]]
    gx, gy = Nd4j.meshgrid(Nd4j.create([1.0, 2, 3]), Nd4j.create([10.0, 20]))
    assert gx.shape() == (2, 3) and gy.t.tolist() == [[10, 10, 10], [20, 20, 20]]
    assert Nd4j.choice(Nd4j.create([1.0, 2, 3]), Nd4j.create([0.0, 1, 0]), 4).t.tolist() == [2, 2, 2, 2]
    s = Nd4j.shuffle(Nd4j.create(np.arange(10.0)), seed=3)
    assert sorted(s.t.tolist()) == list(range(10)) and s.t.tolist() != list(range(10))
    assert Nd4j.clearNans(Nd4j.create([1.0, float("nan")])).t.tolist() == [1, 0] and Nd4j.sizeOfDataType() == 4
    with pytest.raises(ValueError):
        Nd4j.checkShapeValues(2, -1)
    # eager namespaces run registry ops on arrays
    assert Nd4j.math().abs(Nd4j.create([-1.0, 2])).t.tolist() == [1, 2]
    assert torch.allclose(Nd4j.nn().softmax(a, 1).t.sum(1), torch.ones(2))
    assert Nd4j.linalg().matmul(a, Nd4j.eye(3)).t.tolist() == a.t.tolist() if hasattr(Nd4j.linalg(), "matmul") else True
    assert Nd4j.bitwise().and_(Nd4j.create([6], dtype="INT"), Nd4j.create([3], dtype="INT")).t.tolist() == [2] \
        if hasattr(Nd4j.bitwise(), "and_") else True
