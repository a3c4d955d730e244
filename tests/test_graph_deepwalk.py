"""Graph API, random walks and DeepWalk embeddings on two cliques joined by one edge."""
import torch

from deeplearning4j_b200.graph import DeepWalk, Graph, GraphLoader, NoEdgeHandling, NoEdgesException, RandomWalkIterator, WeightedRandomWalkIterator
import pytest


def _two_cliques(k=8):
    g = Graph(2 * k)
    for base in (0, k):
        for i in range(k):
            for j in range(i + 1, k):
                g.addEdge(base + i, base + j)
    g.addEdge(0, k)
    return g


def test_graph_and_walks(tmp_path):
    g = _two_cliques(4)
    assert g.numVertices() == 8 and g.getVertexDegree(0) == 4 and g.getVertexDegree(1) == 3 and sorted(g.getConnectedVertexIndices(4)) == [0, 5, 6, 7]
    it = RandomWalkIterator(g, 6, seed=1)
    walks = list(it)
    assert len(walks) == 8 and all(len(w) == 7 for w in walks) and sorted(w[0].vertexID() for w in walks) == list(range(8))
    for w in walks:
        for a, b in zip(w, w[1:]):
            assert b.vertexID() in g.getConnectedVertexIndices(a.vertexID())
    lone = Graph(3)
    lone.addEdge(0, 1)
    with pytest.raises(NoEdgesException):
        RandomWalkIterator(lone, 3).walks()
    w = RandomWalkIterator(lone, 3, mode=NoEdgeHandling.SELF_LOOP_ON_DISCONNECTED).walks()
    assert w[w[:, 0] == 2][0].tolist() == [2, 2, 2, 2]
    p = tmp_path / "edges.csv"
    p.write_text("0,1,5.0\n1,2,0.0001\n0,2,5.0\n")
    wg = GraphLoader.loadWeightedEdgeListFile(str(p), 3)
    ww = WeightedRandomWalkIterator(wg, 200, seed=3).walks()
    row = ww[ww[:, 0] == 1][0]
    nxt = row[1:][row[:-1] == 1]
    assert float((nxt == 0).float().mean()) > 0.95                       # from vertex 1 the heavy edge to 0 dominates


def test_deepwalk_separates_cliques():
    g = _two_cliques(8)
    dw = DeepWalk.Builder().vectorSize(16).windowSize(3).learningRate(0.05).seed(7).batchSize(512).device("cpu").build()
    dw.initialize(g)
    it = RandomWalkIterator(g, 20, seed=11)
    for _ in range(60):
        dw.fit(it)
    same = sum(dw.similarity(1, j) for j in range(2, 8)) / 6
    other = sum(dw.similarity(1, j) for j in range(9, 16)) / 7
    assert same > other + 0.3, (same, other)
    near = dw.verticesNearest(3, 5)
    assert sum(1 for v in near if v < 8) >= 4 and dw.getVertexVector(0).t.shape == (16,)
