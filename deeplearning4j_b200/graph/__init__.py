"""Graph embeddings (``deeplearning4j-graph``): ``Graph``, random-walk iterators, ``GraphLoader`` and ``DeepWalk``.

DeepWalk (``models/deepwalk/DeepWalk.java``) learns vertex vectors with skip-gram + hierarchical softmax over
truncated random walks; the Huffman tree is built from vertex degrees (``GraphHuffman.java``).  Walks for all
start vertices are generated at once as an index tensor (CSR adjacency, one ``randint`` per step), and the
skip-gram updates reuse the batched trainer of ``nlp.embeddings``.
"""
from __future__ import annotations

import torch

from ..nd.ndarray import INDArray
from ..nlp.embeddings import InMemoryLookupTable, SequenceVectors, VocabCache, VocabWord, build_huffman


class NoEdgeHandling:
    SELF_LOOP_ON_DISCONNECTED = "SELF_LOOP_ON_DISCONNECTED"
    EXCEPTION_ON_DISCONNECTED = "EXCEPTION_ON_DISCONNECTED"


class NoEdgesException(RuntimeError):
    pass


class Vertex:
    def __init__(self, idx, value=None): self.idx, self.value = idx, value
    def vertexID(self): return self.idx
    def getValue(self): return self.value
    def __repr__(self): return f"vertex({self.idx},{self.value})"


class Edge:
    def __init__(self, frm, to, value=None, directed=False): self.frm, self.to, self.value, self.directed = frm, to, value, directed
    def getFrom(self): return self.frm
    def getTo(self): return self.to
    def getValue(self): return self.value
    def isDirected(self): return self.directed


class Graph:
    def __init__(self, numVertices_or_vertices, allowMultipleEdges=False, vertexFactory=None):
        if isinstance(numVertices_or_vertices, int):
            n = numVertices_or_vertices
            self.vertices = [vertexFactory.create(i) if vertexFactory else Vertex(i) for i in range(n)]
        else:
            self.vertices = list(numVertices_or_vertices)
        self.allowMultipleEdges = allowMultipleEdges
        self.adj = [[] for _ in self.vertices]
        self._csr = None

    def numVertices(self): return len(self.vertices)
    def getVertex(self, i): return self.vertices[i]
    def getVertices(self, idx=None): return self.vertices if idx is None else [self.vertices[i] for i in idx]

    def addEdge(self, frm, to=None, value=None, directed=False):
        e = frm if isinstance(frm, Edge) else Edge(frm, to, value, directed)
        if not self.allowMultipleEdges and any(x.to == e.to and x.frm == e.frm for x in self.adj[e.frm]):
            return
        self.adj[e.frm].append(e)
        if not e.directed and e.frm != e.to:
            self.adj[e.to].append(Edge(e.to, e.frm, e.value, False))
        self._csr = None

    def getEdgesOut(self, v): return list(self.adj[v])
    def getVertexDegree(self, v): return len(self.adj[v])
    def getConnectedVertexIndices(self, v): return [e.to for e in self.adj[v]]
    def getConnectedVertices(self, v): return [self.vertices[e.to] for e in self.adj[v]]

    def getRandomConnectedVertex(self, v, rng):
        if not self.adj[v]:
            raise NoEdgesException(f"Cannot generate random connected vertex: vertex {v} has no outgoing/undirected edges")
        return self.vertices[self.adj[v][rng.randrange(len(self.adj[v]))].to]

    def csr(self, device="cpu"):
        if self._csr is None or self._csr[0].device != torch.device(device):
            deg = torch.tensor([len(a) for a in self.adj], dtype=torch.long)
            off = torch.zeros(len(self.adj) + 1, dtype=torch.long)
            off[1:] = deg.cumsum(0)
            nbr = torch.tensor([e.to for a in self.adj for e in a], dtype=torch.long)
            w = torch.tensor([float(e.value) if isinstance(e.value, (int, float)) else 1.0 for a in self.adj for e in a])
            self._csr = (off.to(device), nbr.to(device), deg.to(device), w.to(device))
        return self._csr


class RandomWalkIterator:
    """Uniform random walks of ``walkLength`` steps starting once from every vertex (in shuffled order)."""

    def __init__(self, graph, walkLength, seed=12345, mode=NoEdgeHandling.EXCEPTION_ON_DISCONNECTED, firstVertex=0, lastVertex=None):
        self.graph, self.walkLength, self.seed, self.mode = graph, walkLength, seed, mode
        self.first, self.last = firstVertex, graph.numVertices() if lastVertex is None else lastVertex
        self.epoch = 0
        self.reset()

    def walkLength_(self): return self.walkLength

    def walks(self, device="cpu", weighted=False):
        """All walks of one pass as a [numStarts, walkLength + 1] index tensor."""
        off, nbr, deg, w = self.graph.csr(device)
        g = torch.Generator(device=device).manual_seed(self.seed + self.epoch)
        start = torch.arange(self.first, self.last, device=device)
        start = start[torch.randperm(start.numel(), device=device, generator=g)]
        if self.mode == NoEdgeHandling.EXCEPTION_ON_DISCONNECTED and bool((deg[start] == 0).any()):
            raise NoEdgesException("graph has vertices without outgoing edges")
        out = [start]
        cur = start
        for _ in range(self.walkLength):
            d = deg[cur]
            if weighted:
                # inverse-CDF sampling over each vertex's edge weights (padded to the maximum degree)
                md = int(d.max())
                ar = torch.arange(md, device=device)
                idx = (off[cur].unsqueeze(1) + ar).clamp(max=max(nbr.numel() - 1, 0))
                ww = torch.where(ar.unsqueeze(0) < d.unsqueeze(1), w[idx], torch.zeros((), device=device))
                r = torch.multinomial(ww + (d == 0).unsqueeze(1).float(), 1, generator=g).squeeze(1)
            else:
                r = (torch.rand(cur.numel(), device=device, generator=g) * d.clamp(min=1)).long().clamp(max=(d - 1).clamp(min=0))
            nxt = nbr[(off[cur] + r).clamp(max=max(nbr.numel() - 1, 0))] if nbr.numel() else cur
            cur = torch.where(d > 0, nxt, cur)                        # self loop on disconnected vertices
            out.append(cur)
        return torch.stack(out, 1)

    def reset(self):
        self._walks = None
        self._i = 0

    def hasNext(self):
        if self._walks is None:
            self._walks = self.walks()
        return self._i < self._walks.shape[0]

    def next(self):
        if not self.hasNext():
            raise StopIteration
        row = self._walks[self._i].tolist()
        self._i += 1
        return [self.graph.getVertex(i) for i in row]

    def __iter__(self):
        self.reset()
        while self.hasNext():
            yield self.next()


class WeightedRandomWalkIterator(RandomWalkIterator):
    """Next vertex chosen with probability proportional to the edge weight."""
    def walks(self, device="cpu", weighted=True): return super().walks(device, True)


class GraphLoader:
    @staticmethod
    def loadUndirectedGraphEdgeListFile(path, numVertices, delim=",", allowMultipleEdges=True):
        g = Graph(numVertices, allowMultipleEdges)
        with open(path) as f:
            for line in f:
                line = line.strip()
                if not line or line.startswith("#"):
                    continue
                a, b = line.split(delim)[:2]
                g.addEdge(int(a), int(b), None, False)
        return g

    @staticmethod
    def loadWeightedEdgeListFile(path, numVertices, delim=",", directed=False, allowMultipleEdges=True):
        g = Graph(numVertices, allowMultipleEdges)
        with open(path) as f:
            for line in f:
                p = line.strip().split(delim)
                if len(p) >= 3:
                    g.addEdge(int(p[0]), int(p[1]), float(p[2]), directed)
        return g

    @staticmethod
    def loadGraph(vertexFilePath, edgeFilePath, vertexLoader=None, edgeLineProcessor=None, allowMultipleEdges=True):
        with open(vertexFilePath) as f:
            verts = [(vertexLoader(l.strip()) if vertexLoader else Vertex(i, l.strip())) for i, l in enumerate(f) if l.strip()]
        g = Graph(verts, allowMultipleEdges)
        with open(edgeFilePath) as f:
            for line in f:
                if not line.strip():
                    continue
                e = edgeLineProcessor(line.strip()) if edgeLineProcessor else Edge(*[int(x) for x in line.strip().split(",")[:2]])
                if e is not None:
                    g.addEdge(e)
        return g


class GraphVectors:
    def numVertices(self): return self.lookupTable.syn0.shape[0]
    def getVectorSize(self): return self.vectorSize
    def getVertexVector(self, v): return INDArray(self.lookupTable.syn0[v.vertexID() if isinstance(v, Vertex) else int(v)])

    def similarity(self, a, b):
        va, vb = self.getVertexVector(a).t, self.getVertexVector(b).t
        return float(torch.nn.functional.cosine_similarity(va, vb, dim=0))

    def verticesNearest(self, v, top):
        i = v.vertexID() if isinstance(v, Vertex) else int(v)
        s = self.lookupTable.syn0
        sims = torch.nn.functional.cosine_similarity(s, s[i].unsqueeze(0), dim=1)
        sims[i] = -2.0
        return sims.topk(min(top, s.shape[0] - 1)).indices.tolist()


class DeepWalk(GraphVectors):
    def __init__(self, vectorSize=100, windowSize=2, learningRate=0.01, seed=12345, batchSize=4096, device=None):
        self.vectorSize, self.windowSize, self.learningRate, self.seed, self.batchSize = vectorSize, windowSize, learningRate, seed, batchSize
        self.device = torch.device(device) if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")
        self.lookupTable = None
        self._sv = None

    class Builder:
        def __init__(self): self.kw = {}
        def vectorSize(self, n): self.kw["vectorSize"] = n; return self
        def windowSize(self, n): self.kw["windowSize"] = n; return self
        def learningRate(self, lr): self.kw["learningRate"] = lr; return self
        def seed(self, s): self.kw["seed"] = s; return self
        def batchSize(self, n): self.kw["batchSize"] = n; return self
        def device(self, d): self.kw["device"] = d; return self
        def build(self): return DeepWalk(**self.kw)

    def initialize(self, graph_or_degrees):
        degrees = [graph_or_degrees.getVertexDegree(i) for i in range(graph_or_degrees.numVertices())] \
            if isinstance(graph_or_degrees, Graph) else list(graph_or_degrees)
        vc = VocabCache()
        for i, d in enumerate(degrees):
            vw = VocabWord(str(i), max(d, 1), i)
            vc.words[vw.word] = vw
            vc.by_index.append(vw)
            vc.total += max(d, 1)
        inner = build_huffman(vc)
        sv = SequenceVectors(layerSize=self.vectorSize, windowSize=self.windowSize, learningRate=self.learningRate, minLearningRate=self.learningRate,
                             seed=self.seed, batchSize=self.batchSize, useHierarchicSoftmax=True, negativeSample=0, device=self.device,
                             vocabCache=vc, iterate=[])
        sv.vocab = vc
        sv.lookupTable = InMemoryLookupTable(vc, self.vectorSize, self.seed, self.device, True, 0, inner)
        sv._hs = sv._hs_tables()
        self._sv, self.lookupTable = sv, sv.lookupTable
        return self

    def fit(self, graph_or_iterator, walkLength=None):
        it = graph_or_iterator
        if isinstance(it, Graph):
            if self._sv is None:
                self.initialize(it)
            it = RandomWalkIterator(it, walkLength or 40, self.seed, NoEdgeHandling.SELF_LOOP_ON_DISCONNECTED)
        if self._sv is None:
            self.initialize(it.graph)
        sv = self._sv
        walks = it.walks(self.device)
        it.epoch += 1
        n, L = walks.shape
        ids = walks.reshape(-1)
        sent = torch.arange(n, device=self.device).repeat_interleave(L)
        gen = torch.Generator(device=self.device).manual_seed(self.seed + it.epoch)
        sv._train_elements(ids, sent, gen, lambda done: self.learningRate, [0.0])
        return self
