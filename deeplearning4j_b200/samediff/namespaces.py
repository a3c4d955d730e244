"""SameDiff op namespaces: ``SDBaseOps`` (methods available on the SameDiff instance itself),
``SDMath``, ``SDNN``, ``SDCNN``, ``SDRNN``, ``SDLoss``, ``SDLinalg``, ``SDImage``, ``SDBitwise``,
``SDRandom`` (``nd4j-api/.../autodiff/samediff/ops/*.java``; generated from ``codegen/op-codegen``).

The frequently used methods are spelled out with the reference's argument order; every other
registry op is reachable through a generic fallback: ``sd.math.<camelCaseName>(*variables,
**args)`` resolves to the registry op of the same (camelCase or snake_case) name.  All methods
accept an optional leading ``name`` string like the Java overloads.
"""
from __future__ import annotations

import re

from ..nd.dtype import DataType
from ..ops import registry
from .core import SDVariable


def _snake(n):
    return re.sub(r"(?<!^)(?=[A-Z])", "_", n).lower()


def _split_name(a):
    if a and (isinstance(a[0], str) or a[0] is None) and len(a) > 1 and isinstance(a[1], (SDVariable, list, tuple)):
        return a[0], a[1:]
    return None, a


from ..nd.ndarray import INDArray  # noqa: E402


class _NS:
    ALIASES: dict = {}

    def __init__(self, sd):
        self.sd = sd

    def _o(self, opn, ins, name=None, n_out=None, **kw):
        return self.sd._op(opn, list(ins), n_out=n_out, name=name, **kw)

    def __getattr__(self, item):
        if item.startswith("_"):
            raise AttributeError(item)
        cand = [self.ALIASES.get(item), item, _snake(item), item.lower()]
        opn = next((c for c in cand if c and registry.has(c)), None)
        if opn is None:
            raise AttributeError(f"{type(self).__name__} has no op '{item}'")

        def call(*a, **kw):
            name, a = _split_name(a)
            ins = [x for x in a if isinstance(x, (SDVariable, INDArray)) or x is None]
            extra = [x for x in a if not (isinstance(x, (SDVariable, INDArray)) or x is None)]
            if extra and "dimensions" not in kw and all(isinstance(e, int) for e in extra):
                kw["dimensions"] = list(extra)
            return self._o(opn, ins, name=name, **kw)
        return call


def _dims(d):
    if len(d) == 1 and isinstance(d[0], (list, tuple)):
        return list(d[0])
    return list(d)


class SDBaseOps(_NS):
    ALIASES = {"mmul": "matmul", "oneHot": "onehot", "expandDims": "expand_dims", "gatherNd": "gather_nd",
               "sequenceMask": "sequence_mask", "reverseSequence": "reverse_sequence", "stridedSlice": "strided_slice",
               "dynamicPartition": "dynamic_partition", "dynamicStitch": "dynamic_stitch", "scatterAdd": "scatter_add",
               "scatterUpdate": "scatter_upd", "scatterMul": "scatter_mul", "scatterSub": "scatter_sub", "scatterDiv": "scatter_div",
               "scatterMax": "scatter_max", "scatterMin": "scatter_min", "segmentSum": "segment_sum", "segmentMax": "segment_max",
               "segmentMin": "segment_min", "segmentMean": "segment_mean", "segmentProd": "segment_prod",
               "unsortedSegmentSum": "unsorted_segment_sum", "unsortedSegmentMax": "unsorted_segment_max",
               "unsortedSegmentMin": "unsorted_segment_min", "unsortedSegmentMean": "unsorted_segment_mean",
               "unsortedSegmentProd": "unsorted_segment_prod", "unsortedSegmentSqrtN": "unsorted_segment_sqrt_n",
               "zerosLike": "zeros_as", "onesLike": "ones_as", "linspace": "lin_space", "invertPermutation": "invert_permutation",
               "matchConditionCount": "countNonZero", "normmax": "reduce_norm_max", "squaredNorm": "reduce_sqnorm",
               "standardDeviation": "reduce_stdev", "variance": "reduce_variance", "identity": "identity", "eq": "equals",
               "neq": "not_equals", "gt": "greater", "gte": "greater_equal", "lt": "less", "lte": "less_equal",
               "castTo": "cast", "tensorMmul": "tensormmul", "batchMmul": "batched_gemm", "reshape": "reshape",
               "cumsum": "cumsum", "cumprod": "cumprod", "fill": "fill", "size": "size", "sizeAt": "size_at", "shape": "shape_of",
               "clipByValue": "clipbyvalue", "clipByNorm": "clipbynorm", "assign": "assign", "stopGradient": "stop_gradient"}

    def mmul(self, *a, transposeX=False, transposeY=False, transposeZ=False):
        name, a = _split_name(a)
        return self._o("matmul", a[:2], name=name, transposeX=transposeX, transposeY=transposeY, transposeZ=transposeZ)

    def concat(self, *a):
        name, a = _split_name(a)
        dim = next(x for x in a if isinstance(x, int))
        vs = [x for x in a if isinstance(x, SDVariable)] or list(next(x for x in a if isinstance(x, (list, tuple))))
        return self._o("concat", vs, name=name, concatDimension=dim)

    def stack(self, *a):
        name, a = _split_name(a)
        dim = next((x for x in a if isinstance(x, int)), 0)
        vs = [x for x in a if isinstance(x, SDVariable)] or list(next(x for x in a if isinstance(x, (list, tuple))))
        return self._o("stack", vs, name=name, dimension=dim)

    def unstack(self, *a, num=None):
        name, a = _split_name(a)
        x = next(v for v in a if isinstance(v, SDVariable))
        ints = [v for v in a if isinstance(v, int)]
        axis = ints[0] if ints else 0
        num = ints[1] if len(ints) > 1 else num
        return self._o("unstack", [x], name=name, n_out=num, dimension=axis)

    def split(self, *a):
        name, a = _split_name(a)
        x = next(v for v in a if isinstance(v, SDVariable))
        ints = [v for v in a if isinstance(v, int)]
        return self._o("split", [x], name=name, n_out=ints[0], numSplit=ints[0], dimension=ints[1] if len(ints) > 1 else 0)

    def gather(self, *a, axis=0):
        name, a = _split_name(a)
        vs = [v for v in a if isinstance(v, SDVariable)]
        ints = [v for v in a if isinstance(v, int)]
        return self._o("gather", vs, name=name, axis=ints[0] if ints else axis)

    def reshape(self, *a):
        name, a = _split_name(a)
        x = a[0]
        shape = a[1:] if not isinstance(a[1], (list, tuple, SDVariable)) else a[1]
        if isinstance(shape, SDVariable):
            return self._o("reshape", [x, shape], name=name)
        return self._o("reshape", [x], name=name, shape=[int(s) for s in shape])

    def permute(self, *a):
        name, a = _split_name(a)
        dims = a[1:] if not isinstance(a[1], (list, tuple)) else a[1]
        return self._o("permute", [a[0]], name=name, dimensions=[int(d) for d in dims])

    def transpose(self, *a):
        name, a = _split_name(a)
        return self._o("transpose", [a[0]], name=name)

    def squeeze(self, *a):
        name, a = _split_name(a)
        return self._o("squeeze", [a[0]], name=name, dimensions=[int(a[1])] if len(a) > 1 else None)

    def expandDims(self, *a):
        name, a = _split_name(a)
        return self._o("expand_dims", [a[0]], name=name, axis=int(a[1]))

    def slice(self, *a):
        name, a = _split_name(a)
        return self._o("slice", [a[0]], name=name, begin=list(a[1]), size=list(a[2]))

    def stridedSlice(self, *a, beginMask=0, endMask=0, ellipsisMask=0, newAxisMask=0, shrinkAxisMask=0):
        name, a = _split_name(a)
        return self._o("strided_slice", [a[0]], name=name, begin=list(a[1]), end=list(a[2]), strides=list(a[3]) if len(a) > 3 else None,
                       begin_mask=beginMask, end_mask=endMask, ellipsis_mask=ellipsisMask, new_axis_mask=newAxisMask,
                       shrink_axis_mask=shrinkAxisMask)

    def tile(self, *a):
        name, a = _split_name(a)
        reps = a[1:] if not isinstance(a[1], (list, tuple, SDVariable)) else a[1]
        if isinstance(reps, SDVariable):
            return self._o("tile", [a[0], reps], name=name)
        return self._o("tile", [a[0]], name=name, reps=[int(r) for r in reps])

    def oneHot(self, *a, axis=-1, on=1.0, off=0.0, dataType=DataType.FLOAT):
        name, a = _split_name(a)
        return self._o("onehot", [a[0]], name=name, depth=int(a[1]), axis=int(a[2]) if len(a) > 2 else axis,
                       on=float(a[3]) if len(a) > 3 else on, off=float(a[4]) if len(a) > 4 else off, dtype=int(dataType))

    def castTo(self, *a):
        name, a = _split_name(a)
        return self._o("cast", [a[0]], name=name, dtype=int(a[1]))

    def _reduce(self, opn, a, **kw):
        name, a = _split_name(a)
        x = a[0]
        rest = list(a[1:])
        keep = False
        if rest and isinstance(rest[0], bool):
            keep = rest.pop(0)
        return self._o(opn, [x], name=name, dimensions=_dims(rest), keepDims=keep, **kw)

    def sum(self, *a): return self._reduce("reduce_sum", a)
    def mean(self, *a): return self._reduce("reduce_mean", a)
    def prod(self, *a): return self._reduce("reduce_prod", a)
    def max(self, *a):
        n, b = _split_name(a)
        return self._o("maximum", b[:2], name=n) if len(b) > 1 and isinstance(b[1], SDVariable) else self._reduce("reduce_max", a)
    def min(self, *a):
        n, b = _split_name(a)
        return self._o("minimum", b[:2], name=n) if len(b) > 1 and isinstance(b[1], SDVariable) else self._reduce("reduce_min", a)
    def norm1(self, *a): return self._reduce("reduce_norm1", a)
    def norm2(self, *a): return self._reduce("reduce_norm2", a)
    def argmax(self, *a): return self._reduce("argmax", a)
    def argmin(self, *a): return self._reduce("argmin", a)

    def where(self, *a):
        name, a = _split_name(a)
        if len(a) == 3:
            return self._o("select", [a[2], a[0], a[1]] if False else [a[0], a[1], a[2]], name=name)
        return self._o("Where", a, name=name)

    def range(self, *a, dataType=DataType.FLOAT):
        name, a = (a[0], a[1:]) if a and isinstance(a[0], str) else (None, a)
        nums = [v for v in a if not isinstance(v, DataType)]
        dt = next((v for v in a if isinstance(v, DataType)), dataType)
        return self._o("range", [], name=name, frm=nums[0], to=nums[1], step=nums[2] if len(nums) > 2 else 1, dtype=int(dt))


class SDMath(_NS):
    ALIASES = {"log1p": "log1p", "rsqrt": "rsqrt", "isNaN": "isnan", "isInfinite": "isinf", "isFinite": "isfinite",
               "cosineSimilarity": "cosinesimilarity", "cosineDistance": "cosinedistance", "euclideanDistance": "euclidean",
               "manhattanDistance": "manhattan", "hammingDistance": "hammingdistance", "jaccardDistance": "jaccarddistance",
               "clipByValue": "clipbyvalue", "clipByNorm": "clipbynorm", "confusionMatrix": "confusion_matrix",
               "logSumExp": "reduce_logsumexp", "standardize": "standardize", "squaredDifference": "squaredsubtract",
               "floorDiv": "floordiv", "floorMod": "floormod", "firstIndex": "firstindex", "lastIndex": "lastindex",
               "iamax": "argamax", "iamin": "argamin", "countNonZero": "countNonZero", "countZero": "countZero",
               "mergeAdd": "mergeadd", "mergeAvg": "mergeavg", "mergeMax": "mergemax", "setDiag": "matrix_set_diag",
               "diagPart": "diag_part", "atan2": "tf_atan2", "and": "boolean_and", "or": "boolean_or", "xor": "boolean_xor",
               "add": "add", "sub": "subtract", "mul": "multiply", "div": "divide", "rsub": "reversesubtract", "rdiv": "reversedivide",
               "pow": "pow", "cube": "cube", "square": "square", "entropy": "entropy", "logEntropy": "log_entropy",
               "shannonEntropy": "shannonentropy", "amax": "amax", "amin": "amin", "amean": "amean", "asum": "asum",
               "zeroFraction": "zero_fraction", "isMax": "ismax", "listDiff": "listdiff", "meshgrid": "meshgrid",
               "moments": "moments", "normalizeMoments": "normalize_moments", "bitShift": "shift_bits", "bitShiftRight": "rshift_bits"}

    def pow(self, *a):
        name, a = _split_name(a)
        if isinstance(a[1], SDVariable):
            return self._o("Pow", a[:2], name=name)
        return self._o("pow", [a[0]], name=name, p=float(a[1]))


class SDNN(_NS):
    ALIASES = {"leakyRelu": "lrelu", "hardTanh": "hardtanh", "hardSigmoid": "hardsigmoid", "softsign": "softsign",
               "softplus": "softplus", "logSoftmax": "log_softmax", "biasAdd": "biasadd", "batchNorm": "batchnorm",
               "reluLayer": "relu_layer", "preciseGelu": "precise_gelu", "logSigmoid": "logsigmoid", "pad": "pad",
               "topK": "top_k", "cReLU": "crelu"}

    def linear(self, *a):
        name, a = _split_name(a)
        return self._o("xw_plus_b", [a[0], a[1], a[2] if len(a) > 2 else None], name=name)

    def reluLayer(self, *a):
        name, a = _split_name(a)
        return self._o("relu_layer", a[:3], name=name)

    def softmax(self, *a, dimension=-1):
        name, a = _split_name(a)
        return self._o("softmax", [a[0]], name=name, dimension=int(a[1]) if len(a) > 1 else dimension)

    def logSoftmax(self, *a, dimension=-1):
        name, a = _split_name(a)
        return self._o("log_softmax", [a[0]], name=name, dimension=int(a[1]) if len(a) > 1 else dimension)

    def layerNorm(self, *a):
        name, a = _split_name(a)
        vs = [v for v in a if isinstance(v, SDVariable)]
        rest = [v for v in a if not isinstance(v, SDVariable)]
        ch_first = rest[0] if rest and isinstance(rest[0], bool) else False
        dims = [v for v in rest if isinstance(v, int) and not isinstance(v, bool)] or [-1]
        return self._o("layer_norm", [vs[0], vs[1], vs[2] if len(vs) > 2 else None], name=name, dimensions=dims, channelsFirst=ch_first)

    def dropout(self, *a):
        name, a = _split_name(a)
        return self._o("dropout", [a[0]], name=name, probValue=float(a[1]))

    def relu(self, *a):
        name, a = _split_name(a)
        return self._o("relu", [a[0]], name=name, cutoff=float(a[1]) if len(a) > 1 else 0.0)

    def leakyRelu(self, *a):
        name, a = _split_name(a)
        return self._o("lrelu", [a[0]], name=name, alpha=float(a[1]) if len(a) > 1 else 0.01)

    def elu(self, *a):
        name, a = _split_name(a)
        return self._o("elu", [a[0]], name=name)

    def batchNorm(self, *a, epsilon=1e-5):
        name, a = _split_name(a)
        vs = [v for v in a if isinstance(v, SDVariable)]
        rest = [v for v in a if not isinstance(v, SDVariable)]
        eps = next((v for v in rest if isinstance(v, float)), epsilon)
        axis = [v for v in rest if isinstance(v, int)] or [1]
        return self._o("batchnorm", vs + [None] * (5 - len(vs)), name=name, epsilon=eps, axis=axis)

    def dotProductAttention(self, *a, scaled=True, withWeights=False):
        name, a = _split_name(a)
        vs = list(a[:4]) + [None] * (4 - len(a[:4]))
        flags = [v for v in a if isinstance(v, bool)]
        vs = [v if isinstance(v, SDVariable) else None for v in vs]
        scaled = flags[0] if flags else scaled
        withWeights = flags[1] if len(flags) > 1 else withWeights
        r = self._o("dot_product_attention", vs, name=name, n_out=2 if withWeights else 1, scaled=scaled, withWeights=withWeights)
        return r

    def dotProductAttentionV2(self, *a, scale=1.0, dropoutProbability=0.0, useCausalMask=False, training=False):
        name, a = _split_name(a)
        vs = [v if isinstance(v, SDVariable) else None for v in a[:6]]
        vs += [None] * (6 - len(vs))
        return self._o("dot_product_attention_v2", vs, name=name, n_out=1, scale=scale, dropoutProbability=dropoutProbability,
                       useCausalMask=useCausalMask)

    def multiHeadDotProductAttention(self, *a, scaled=True, withWeights=False):
        name, a = _split_name(a)
        vs = [v if isinstance(v, SDVariable) else None for v in a[:8]]
        vs += [None] * (8 - len(vs))
        flags = [v for v in a if isinstance(v, bool)]
        return self._o("multi_head_dot_product_attention", vs, name=name, n_out=1, scaled=flags[0] if flags else scaled)


class SDCNN(_NS):
    ALIASES = {"avgPooling2d": "avgpool2d", "maxPooling2d": "maxpool2d", "avgPooling3d": "avgpool3dnew", "maxPooling3d": "maxpool3dnew",
               "conv3d": "conv3dnew", "depthWiseConv2d": "depthwise_conv2d", "separableConv2d": "sconv2d", "im2Col": "im2col",
               "col2Im": "col2im", "batchToSpace": "batch_to_space", "spaceToBatch": "space_to_batch", "depthToSpace": "depth_to_space",
               "spaceToDepth": "space_to_depth", "upsampling2d": "upsampling2d", "upsampling3d": "upsampling3d",
               "localResponseNormalization": "lrn", "extractImagePatches": "extract_image_patches",
               "maxPoolWithArgmax": "max_pool_with_argmax", "dilation2D": "dilation2d"}

    @staticmethod
    def _cfg(cfg):
        if cfg is None:
            return {}
        d = dict(cfg) if isinstance(cfg, dict) else {k: v for k, v in vars(cfg).items() if not k.startswith("_")}
        if "dataFormat" in d and isinstance(d["dataFormat"], str):
            d["dataFormat"] = 1 if d["dataFormat"].upper() in ("NHWC", "NWC", "NDHWC") else 0
        return d

    def _conv(self, opn, a, **kw):
        name, a = _split_name(a)
        vs = [v for v in a if isinstance(v, SDVariable) or v is None]
        cfg = next((v for v in a if not isinstance(v, (SDVariable, str)) and v is not None), None)
        args = self._cfg(cfg)
        args.update(kw)
        return self._o(opn, vs, name=name, **args)

    def conv2d(self, *a, **kw): return self._conv("conv2d", a, **kw)
    def conv1d(self, *a, **kw): return self._conv("conv1d", a, **kw)
    def conv3d(self, *a, **kw): return self._conv("conv3dnew", a, **kw)
    def deconv2d(self, *a, **kw): return self._conv("deconv2d", a, **kw)
    def deconv3d(self, *a, **kw): return self._conv("deconv3d", a, **kw)
    def depthWiseConv2d(self, *a, **kw): return self._conv("depthwise_conv2d", a, **kw)
    def separableConv2d(self, *a, **kw): return self._conv("sconv2d", a, **kw)
    def maxPooling2d(self, *a, **kw): return self._conv("maxpool2d", a, **kw)
    def avgPooling2d(self, *a, **kw): return self._conv("avgpool2d", a, **kw)
    def maxPooling3d(self, *a, **kw): return self._conv("maxpool3dnew", a, **kw)
    def avgPooling3d(self, *a, **kw): return self._conv("avgpool3dnew", a, **kw)


class Conv2DConfig:
    def __init__(self, kH=1, kW=1, sH=1, sW=1, pH=0, pW=0, dH=1, dW=1, isSameMode=False, dataFormat="NCHW", wFormat=0, paddingMode=None):
        self.kH, self.kW, self.sH, self.sW, self.pH, self.pW, self.dH, self.dW = kH, kW, sH, sW, pH, pW, dH, dW
        self.isSameMode, self.dataFormat, self.wFormat, self.paddingMode = isSameMode, dataFormat, wFormat, paddingMode


Pooling2DConfig = Conv2DConfig


class Conv1DConfig:
    def __init__(self, k=1, s=1, p=0, d=1, isSameMode=False, dataFormat="NCW", paddingMode=None, wFormat=0):
        self.k, self.s, self.p, self.d, self.isSameMode, self.dataFormat, self.paddingMode, self.wFormat = k, s, p, d, isSameMode, dataFormat, paddingMode, wFormat


class Conv3DConfig:
    def __init__(self, kD=1, kH=1, kW=1, sD=1, sH=1, sW=1, pD=0, pH=0, pW=0, dD=1, dH=1, dW=1, isSameMode=False, dataFormat="NCDHW", wFormat=0):
        self.__dict__.update(dict(kD=kD, kH=kH, kW=kW, sD=sD, sH=sH, sW=sW, pD=pD, pH=pH, pW=pW, dD=dD, dH=dH, dW=dW,
                                  isSameMode=isSameMode, wFormat=wFormat))
        self.dataFormat = 0 if str(dataFormat).upper() == "NCDHW" else 1


class SDRNN(_NS):
    ALIASES = {"lstmLayer": "lstmLayer", "lstmCell": "lstmLayerCell", "gru": "gru", "gruCell": "gruCell", "sru": "sru", "sruCell": "sruCell",
               "lstmblock": "lstmBlock"}

    def lstmLayer(self, *a, n_out=None, **cfg):
        name, a = _split_name(a)
        vs = [v if isinstance(v, SDVariable) else None for v in a[:8]]
        vs += [None] * (8 - len(vs))
        n = int(bool(cfg.get("retFullSeq", True))) + int(bool(cfg.get("retLastH", False))) + int(bool(cfg.get("retLastC", False)))
        return self._o("lstmLayer", vs, name=name, n_out=n_out or max(n, 1), **cfg)


class SDLoss(_NS):
    ALIASES = {"absoluteDifference": "absolute_difference_loss", "cosineDistance": "cosine_distance_loss", "hingeLoss": "hinge_loss",
               "huberLoss": "huber_loss", "l2Loss": "l2_loss", "logLoss": "log_loss", "logPoisson": "log_poisson_loss",
               "meanPairwiseSquaredError": "mean_pairwssqerr_loss", "meanSquaredError": "mean_sqerr_loss",
               "sigmoidCrossEntropy": "sigm_cross_entropy_loss", "softmaxCrossEntropy": "softmax_cross_entropy_loss",
               "sparseSoftmaxCrossEntropy": "sparse_softmax_cross_entropy_loss_with_logits",
               "weightedCrossEntropyWithLogits": "weighted_cross_entropy_with_logits", "ctcLoss": "ctc_loss"}

    def _loss(self, opn, a, **kw):
        """(name?, label, predictions, weights?, lossReduce?) -> native order (predictions, weights, labels)."""
        name = None
        if a and isinstance(a[0], str):
            name, a = a[0], a[1:]
        vs = [v for v in a if isinstance(v, SDVariable) or v is None]
        red = next((v for v in a if isinstance(v, (int, str)) and not isinstance(v, bool)), 3)
        label, pred = vs[0], vs[1]
        w = vs[2] if len(vs) > 2 else None
        out = self._o(opn, [pred, w, label], name=name, reductionMode=red, **kw)
        out.markAsLoss()
        return out

    def meanSquaredError(self, *a): return self._loss("mean_sqerr_loss", a)
    def absoluteDifference(self, *a): return self._loss("absolute_difference_loss", a)
    def hingeLoss(self, *a): return self._loss("hinge_loss", a)
    def huberLoss(self, *a, delta=1.0): return self._loss("huber_loss", a, delta=delta)
    def logLoss(self, *a, epsilon=1e-7): return self._loss("log_loss", a, epsilon=epsilon)
    def logPoisson(self, *a, full=False): return self._loss("log_poisson_loss", a, full=full)
    def sigmoidCrossEntropy(self, *a, labelSmoothing=0.0): return self._loss("sigm_cross_entropy_loss", a, labelsSmoothing=labelSmoothing)
    def softmaxCrossEntropy(self, *a, labelSmoothing=0.0): return self._loss("softmax_cross_entropy_loss", a, labelsSmoothing=labelSmoothing)
    def meanPairwiseSquaredError(self, *a): return self._loss("mean_pairwssqerr_loss", a)
    def cosineDistance(self, *a, dimension=-1): return self._loss("cosine_distance_loss", a, dimension=dimension)

    def sparseSoftmaxCrossEntropy(self, *a):
        name = None
        if a and isinstance(a[0], str):
            name, a = a[0], a[1:]
        logits, labels = a[0], a[1]
        per = self._o("sparse_softmax_cross_entropy_loss_with_logits", [labels, logits])
        out = self._o("reduce_mean", [per], name=name, dimensions=[], keepDims=False)
        out.markAsLoss()
        return out

    def l2Loss(self, *a):
        name, a = _split_name(a) if len(a) > 1 else (None, a)
        out = self._o("l2_loss", [a[-1]], name=name)
        out.markAsLoss()
        return out


class SDLinalg(_NS):
    ALIASES = {"cholesky": "cholesky", "lstsq": "lstsq", "solve": "solve", "triangularSolve": "triangular_solve", "lu": "lu",
               "matmul": "matmul", "qr": "qr", "svd": "svd", "logdet": "logdet", "matrixBandPart": "matrix_band_part",
               "cross": "cross", "diag": "diag", "diagPart": "diag_part", "mmul": "matmul", "tri": "tri", "triu": "triu",
               "matrixDeterminant": "matrix_determinant", "matrixInverse": "matrix_inverse", "eig": "eig"}


class SDImage(_NS):
    ALIASES = {"cropAndResize": "crop_and_resize", "adjustContrast": "adjust_contrast", "adjustHue": "adjust_hue",
               "adjustSaturation": "adjust_saturation", "extractImagePatches": "extract_image_patches", "hsvToRgb": "hsv_to_rgb",
               "rgbToHsv": "rgb_to_hsv", "rgbToYiq": "rgb_to_yiq", "rgbToYuv": "rgb_to_yuv", "yiqToRgb": "yiq_to_rgb",
               "yuvToRgb": "yuv_to_rgb", "imageResize": "image_resize", "nonMaxSuppression": "non_max_suppression",
               "randomCrop": "random_crop", "resizeBiLinear": "resize_bilinear", "resizeBiCubic": "resize_bicubic",
               "resizeNearestNeighbor": "resize_nearest_neighbor", "resizeArea": "resize_area"}


class SDBitwise(_NS):
    ALIASES = {"and": "bitwise_and", "or": "bitwise_or", "xor": "bitwise_xor", "leftShift": "shift_bits", "rightShift": "rshift_bits",
               "leftShiftCyclic": "cyclic_shift_bits", "rightShiftCyclic": "cyclic_rshift_bits",
               "bitsHammingDistance": "bits_hamming_distance", "bitRotl": "cyclic_shift_bits", "bitRotr": "cyclic_rshift_bits",
               "bitShift": "shift_bits", "bitShiftRight": "rshift_bits", "toggleBits": "toggle_bits"}


class SDRandom(_NS):
    def _r(self, opn, name, shape, dtype, **kw):
        return self._o(opn, [], name=name, shape=[int(s) for s in shape], dtype=int(dtype), **kw)

    @staticmethod
    def _parse(a):
        name = a[0] if a and isinstance(a[0], str) else None
        a = a[1:] if name is not None else a
        nums = [v for v in a if isinstance(v, (int, float)) and not isinstance(v, (bool, DataType))]
        dt = next((v for v in a if isinstance(v, DataType)), DataType.FLOAT)
        shape = next((v for v in a if isinstance(v, (list, tuple))), None)
        return name, nums, dt, shape

    def uniform(self, *a):
        name, nums, dt, shape = self._parse(a)
        shape = shape if shape is not None else nums[2:]
        return self._r("randomuniform", name, shape, dt, min=float(nums[0]), max=float(nums[1]))

    def normal(self, *a):
        name, nums, dt, shape = self._parse(a)
        shape = shape if shape is not None else nums[2:]
        return self._r("random_normal", name, shape, dt, mean=float(nums[0]), stdev=float(nums[1]))

    def bernoulli(self, *a):
        name, nums, dt, shape = self._parse(a)
        shape = shape if shape is not None else nums[1:]
        return self._r("random_bernoulli", name, shape, dt, p=float(nums[0]))

    def exponential(self, *a):
        name, nums, dt, shape = self._parse(a)
        shape = shape if shape is not None else nums[1:]
        return self._r("random_exponential", name, shape, dt, lambda_=float(nums[0]))

    def logNormal(self, *a):
        name, nums, dt, shape = self._parse(a)
        shape = shape if shape is not None else nums[2:]
        return self._r("distribution_lognormal", name, shape, dt, mean=float(nums[0]), stdev=float(nums[1]))

    def normalTruncated(self, *a):
        name, nums, dt, shape = self._parse(a)
        shape = shape if shape is not None else nums[2:]
        return self._r("distribution_truncated", name, shape, dt, mean=float(nums[0]), stdev=float(nums[1]))

    def binomial(self, *a):
        name, nums, dt, shape = self._parse(a)
        shape = shape if shape is not None else nums[2:]
        return self._r("distribution_binomial", name, shape, dt, trials=int(nums[0]), p=float(nums[1]))


class EagerOps:
    """Stands in for a ``SameDiff`` instance behind the namespace classes and runs every op at once on arrays: this is what
    ``Nd4j.math() / nn() / cnn() / rnn() / loss() / linalg() / image() / bitwise() / random()`` return
    (``nd4j-api/.../linalg/factory/ops/ND*.java`` are the eager twins of the ``SD*`` namespaces)."""

    def _op(self, opn, ins, n_out=None, name=None, **kw):
        import torch
        args = [x.t if isinstance(x, INDArray) else x for x in ins]
        out = registry.get(opn).fn(*args, **kw)
        if isinstance(out, (tuple, list)):
            return [INDArray(o) if isinstance(o, torch.Tensor) else o for o in out]
        return INDArray(out) if isinstance(out, torch.Tensor) else out
