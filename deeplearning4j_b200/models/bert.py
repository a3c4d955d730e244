"""BERT-shaped encoder with a masked-LM head as a SameDiff graph.

The reference ships only the data side of BERT (``deeplearning4j-nlp/.../iterator/BertIterator.java``,
``BertMaskedLMMasker`` with 15 % masking) and imports the model through TF/ONNX; this builder
defines the same architecture natively through the SameDiff API (``sd.var`` / ``sd.nn.linear`` /
``sd.nn.layerNorm`` / ``sd.nn.dotProductAttentionV2`` / ``sd.loss.sparseSoftmaxCrossEntropy``).

Placeholders: ``tokens`` [B, T] int64, ``maskedPositions`` [nMasked] int64 (flat indices into
B*T), ``maskedLabels`` [nMasked] int64 and optionally ``attentionMask`` [B, T].  Activations are kept
as [B*T, hidden] matrices so that every projection is one GEMM.
"""
from __future__ import annotations

from dataclasses import dataclass

from ..nd.dtype import DataType
from ..nn.weights import NormalDistribution, WeightInitDistribution, WeightInitZero
from ..samediff.core import SameDiff
from ..samediff.training import TrainingConfig


@dataclass
class BertConfig:
    vocabSize: int = 30522
    hidden: int = 768
    layers: int = 12
    heads: int = 12
    ffn: int = 3072
    maxPositions: int = 512
    typeVocab: int = 2
    layerNormEps: float = 1e-5
    initStd: float = 0.02
    useAttentionMask: bool = False

    @staticmethod
    def base():
        return BertConfig()

    @staticmethod
    def tiny():
        return BertConfig(vocabSize=1000, hidden=64, layers=2, heads=4, ffn=128, maxPositions=64)


def build_bert_mlm(cfg: BertConfig, batch: int, seqLen: int, updater=None, computeDataType: DataType | None = None) -> SameDiff:
    sd = SameDiff.create()
    H, nh = cfg.hidden, cfg.heads
    dh = H // nh
    w = WeightInitDistribution(NormalDistribution(0.0, cfg.initStd))
    one, zero = WeightInitZero(1.0), WeightInitZero(0.0)

    tokens = sd.placeHolder("tokens", DataType.LONG, batch, seqLen)
    positions = sd.placeHolder("maskedPositions", DataType.LONG, -1)
    labels = sd.placeHolder("maskedLabels", DataType.LONG, -1)
    amask = sd.placeHolder("attentionMask", DataType.FLOAT, batch, seqLen) if cfg.useAttentionMask else None

    wordEmb = sd.var("embeddings/word", w, DataType.FLOAT, cfg.vocabSize, H)
    posEmb = sd.var("embeddings/position", w, DataType.FLOAT, cfg.maxPositions, H)
    embG = sd.var("embeddings/ln_gamma", one, DataType.FLOAT, H)
    embB = sd.var("embeddings/ln_beta", zero, DataType.FLOAT, H)

    x = sd.gather("embeddings/lookup", wordEmb, sd.reshape(tokens, -1), 0)                 # [B*T, H]
    pos = sd.tile(sd.stridedSlice(posEmb, [0, 0], [seqLen, H], [1, 1]), batch, 1)          # [B*T, H]
    x = sd.nn.layerNorm("embeddings/ln", x.add(pos), embG, embB, False, 1)

    for l in range(cfg.layers):
        p = f"layer{l}/"
        Wqkv = sd.var(p + "attn/Wqkv", w, DataType.FLOAT, H, 3 * H)
        bqkv = sd.var(p + "attn/bqkv", zero, DataType.FLOAT, 3 * H)
        Wo = sd.var(p + "attn/Wo", w, DataType.FLOAT, H, H)
        bo = sd.var(p + "attn/bo", zero, DataType.FLOAT, H)
        g1 = sd.var(p + "ln1_gamma", one, DataType.FLOAT, H)
        b1 = sd.var(p + "ln1_beta", zero, DataType.FLOAT, H)
        W1 = sd.var(p + "ffn/W1", w, DataType.FLOAT, H, cfg.ffn)
        bf1 = sd.var(p + "ffn/b1", zero, DataType.FLOAT, cfg.ffn)
        W2 = sd.var(p + "ffn/W2", w, DataType.FLOAT, cfg.ffn, H)
        bf2 = sd.var(p + "ffn/b2", zero, DataType.FLOAT, H)
        g2 = sd.var(p + "ln2_gamma", one, DataType.FLOAT, H)
        b2 = sd.var(p + "ln2_beta", zero, DataType.FLOAT, H)

        qkv = sd.nn.linear(p + "attn/qkv", x, Wqkv, bqkv)                                   # [B*T, 3H]
        qkv5 = sd.reshape(qkv, batch, seqLen, 3, nh, dh)
        q, k, v = sd.unstack(qkv5, 2, 3)                                                    # each [B, T, nh, dh]
        q, k, v = (sd.permute(t, 0, 2, 1, 3) for t in (q, k, v))                            # [B, nh, T, dh]
        att = sd.nn.dotProductAttentionV2(p + "attn/sdpa", q, v, k, None, None, amask, scale=dh ** -0.5)
        ctxv = sd.reshape(sd.permute(att, 0, 2, 1, 3), batch * seqLen, H)
        proj = sd.nn.linear(p + "attn/out", ctxv, Wo, bo)
        x = sd.nn.layerNorm(p + "ln1", x.add(proj), g1, b1, False, 1)
        h = sd.nn.gelu(sd.nn.linear(p + "ffn/in", x, W1, bf1))
        h = sd.nn.linear(p + "ffn/out", h, W2, bf2)
        x = sd.nn.layerNorm(p + "ln2", x.add(h), g2, b2, False, 1)

    # masked-LM head on the gathered positions only (15 % of the tokens)
    Wt = sd.var("mlm/transform_W", w, DataType.FLOAT, H, H)
    bt = sd.var("mlm/transform_b", zero, DataType.FLOAT, H)
    gt = sd.var("mlm/ln_gamma", one, DataType.FLOAT, H)
    btl = sd.var("mlm/ln_beta", zero, DataType.FLOAT, H)
    # The decoder is padded to a multiple of 8 classes so that its rows are 16-byte aligned for TMA; the pad
    # classes have zero weights and a large negative bias, i.e. zero probability mass and zero gradient.
    vpad = (cfg.vocabSize + 7) // 8 * 8
    import torch
    g = torch.Generator().manual_seed(12345)
    wdec0 = torch.zeros(H, vpad)
    wdec0[:, :cfg.vocabSize].normal_(0.0, cfg.initStd, generator=g)
    bdec0 = torch.zeros(vpad)
    bdec0[cfg.vocabSize:] = -30000.0
    Wdec = sd.var("mlm/decoder_W", wdec0)
    bdec = sd.var("mlm/decoder_b", bdec0)
    hm = sd.gather("mlm/gather", x, positions, 0)
    hm = sd.nn.layerNorm("mlm/ln", sd.nn.gelu(sd.nn.linear("mlm/transform", hm, Wt, bt)), gt, btl, False, 1)
    logits = sd.nn.linear("mlm/logits", hm, Wdec, bdec)
    loss = sd.loss.sparseSoftmaxCrossEntropy("loss", logits, labels)
    sd.setLossVariables(loss)

    from ..nn.updaters import Adam
    tcb = (TrainingConfig.builder().updater(updater or Adam(1e-4))
           .dataSetFeatureMapping(*(["tokens", "maskedPositions"] + (["attentionMask"] if amask is not None else [])))
           .dataSetLabelMapping("maskedLabels"))
    if computeDataType is not None:
        tcb.computeDataType(computeDataType)
    sd.setTrainingConfig(tcb.build())
    return sd
