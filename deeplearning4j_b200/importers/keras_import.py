"""Keras model import (``deeplearning4j-modelimport``: ``KerasModelImport``, ``KerasSequentialModel``, ``KerasModel``
and the ``Keras*`` layer mappers).  A model is its architecture JSON (``model.to_json()`` / the ``model_config``
attribute of an HDF5 file) plus weights.  Weights come from a ``{layer name: [arrays]}`` dict, an ``.npz`` file
with ``<layer>/<index>`` keys, or an HDF5 file read by ``importers/hdf5.py`` (no HDF5 library is needed); a full-model ``.h5``
file passed as the first argument supplies both.  Sequential models become a ``MultiLayerNetwork``, functional models a
``ComputationGraph``; Keras channels-last tensors map onto the NCHW layers by permuting kernels at import time and
inserting the flatten order fix for ``Flatten`` -> ``Dense``."""
from __future__ import annotations

import json

import numpy as np
import torch

from .. import nn
from ..nn.conf.graphconf import ElementWiseVertex, MergeVertex
from ..nn.conf.graphconf import PreprocessorVertex
from ..nn.conf.preprocessors import CnnToFeedForwardPreProcessor, ComposableInputPreProcessor, PermutePreprocessor, ReshapePreprocessor

_LAMBDA_LAYERS = {}          # Keras Lambda layer name -> layer (KerasLayer.registerLambdaLayer)
_CUSTOM_LAYERS = {}          # Keras class name -> callable(config) -> layer (KerasLayer.registerCustomLayer)

_ACT = {"relu": "RELU", "sigmoid": "SIGMOID", "tanh": "TANH", "softmax": "SOFTMAX", "linear": "IDENTITY", None: "IDENTITY", "elu": "ELU", "selu": "SELU",
        "softplus": "SOFTPLUS", "softsign": "SOFTSIGN", "hard_sigmoid": "HARDSIGMOID", "swish": "SWISH", "gelu": "GELU", "leaky_relu": "LEAKYRELU", "relu6": "RELU6"}
_LOSS = {"categorical_crossentropy": "MCXENT", "sparse_categorical_crossentropy": "SPARSE_MCXENT", "binary_crossentropy": "XENT", "mse": "MSE",
         "mean_squared_error": "MSE", "mae": "MEAN_ABSOLUTE_ERROR", "mean_absolute_error": "MEAN_ABSOLUTE_ERROR", "kullback_leibler_divergence": "KL_DIVERGENCE",
         "hinge": "HINGE", "squared_hinge": "SQUARED_HINGE", "poisson": "POISSON", "cosine_proximity": "COSINE_PROXIMITY"}


class InvalidKerasConfigurationException(ValueError):
    pass


class UnsupportedKerasConfigurationException(NotImplementedError):
    pass


def _act(cfg):
    a = cfg.get("activation")
    if isinstance(a, dict):
        a = a.get("class_name", "linear").lower()
    if a not in _ACT:
        raise UnsupportedKerasConfigurationException(f"Unsupported Keras activation: {a}")
    return _ACT[a]


def _pair(v):
    return [int(v), int(v)] if isinstance(v, int) else [int(x) for x in v]


def _triple(v):
    return [int(v)] * 3 if isinstance(v, int) else [int(x) for x in v]


def _sides(v, n):
    """Keras padding / cropping argument -> flat [before, after] * n."""
    if isinstance(v, int):
        return [int(v)] * (2 * n)
    out = []
    for e in v:
        out += [int(e), int(e)] if isinstance(e, int) else [int(e[0]), int(e[1])]
    return out


def _mode(cfg):
    return "Same" if str(cfg.get("padding", "valid")).lower() == "same" else "Truncate"


def _map_layer(cls, cfg, is_last, loss):
    """-> (layer or None, kind) where kind in {'layer', 'flatten', 'input', 'skip', 'merge-add', 'merge-concat', ...}."""
    name = cfg.get("name")
    if cls == "InputLayer":
        return None, "input"
    if cls == "Dense":
        if is_last and loss:
            return nn.OutputLayer(loss, nOut=cfg["units"], activation=_act(cfg), hasBias=cfg.get("use_bias", True), layerName=name), "layer"
        return nn.DenseLayer(nOut=cfg["units"], activation=_act(cfg), hasBias=cfg.get("use_bias", True), layerName=name), "layer"
    if cls in ("Conv2D", "Convolution2D"):
        return nn.ConvolutionLayer(_pair(cfg["kernel_size"]), _pair(cfg.get("strides", 1)), nOut=cfg["filters"], activation=_act(cfg), convolutionMode=_mode(cfg),
                                   dilation=_pair(cfg.get("dilation_rate", 1)), hasBias=cfg.get("use_bias", True), layerName=name), "layer"
    if cls in ("Conv1D", "Convolution1D"):
        k = cfg["kernel_size"][0] if isinstance(cfg["kernel_size"], (list, tuple)) else cfg["kernel_size"]
        s = cfg.get("strides", 1)
        s = s[0] if isinstance(s, (list, tuple)) else s
        return nn.Convolution1DLayer([int(k)], [int(s)], nOut=cfg["filters"], activation=_act(cfg), convolutionMode=_mode(cfg), hasBias=cfg.get("use_bias", True), layerName=name), "layer"
    if cls == "SeparableConv2D":
        return nn.SeparableConvolution2D(_pair(cfg["kernel_size"]), _pair(cfg.get("strides", 1)), nOut=cfg["filters"], activation=_act(cfg), convolutionMode=_mode(cfg),
                                         depthMultiplier=cfg.get("depth_multiplier", 1), hasBias=cfg.get("use_bias", True), layerName=name), "layer"
    if cls == "DepthwiseConv2D":
        return nn.DepthwiseConvolution2D(_pair(cfg["kernel_size"]), _pair(cfg.get("strides", 1)), activation=_act(cfg), convolutionMode=_mode(cfg),
                                         depthMultiplier=cfg.get("depth_multiplier", 1), hasBias=cfg.get("use_bias", True), layerName=name), "layer"
    if cls in ("Conv2DTranspose", "Deconvolution2D"):
        return nn.Deconvolution2D(_pair(cfg["kernel_size"]), _pair(cfg.get("strides", 1)), nOut=cfg["filters"], activation=_act(cfg), convolutionMode=_mode(cfg),
                                  hasBias=cfg.get("use_bias", True), layerName=name), "layer"
    if cls in ("MaxPooling2D", "AveragePooling2D"):
        ps = _pair(cfg.get("pool_size", 2))
        return nn.SubsamplingLayer("MAX" if cls.startswith("Max") else "AVG", ps, _pair(cfg.get("strides") or ps), convolutionMode=_mode(cfg), layerName=name), "layer"
    if cls in ("MaxPooling1D", "AveragePooling1D"):
        ps = cfg.get("pool_size", 2)
        ps = ps[0] if isinstance(ps, (list, tuple)) else ps
        st = cfg.get("strides") or ps
        st = st[0] if isinstance(st, (list, tuple)) else st
        return nn.Subsampling1DLayer("MAX" if cls.startswith("Max") else "AVG", [int(ps)], [int(st)], convolutionMode=_mode(cfg), layerName=name), "layer"
    if cls in ("GlobalAveragePooling2D", "GlobalMaxPooling2D", "GlobalAveragePooling1D", "GlobalMaxPooling1D"):
        return nn.GlobalPoolingLayer("AVG" if "Average" in cls else "MAX", layerName=name), "layer"
    if cls == "Flatten":
        return None, "flatten"
    if cls == "Dropout":
        return nn.DropoutLayer(1.0 - float(cfg.get("rate", 0.5)), layerName=name), "layer"        # DL4J stores the retain probability
    if cls in ("SpatialDropout1D", "SpatialDropout2D", "SpatialDropout3D"):
        return nn.DropoutLayer(nn.SpatialDropout(1.0 - float(cfg.get("rate", 0.5))), layerName=name), "layer"
    if cls == "AlphaDropout":
        return nn.DropoutLayer(nn.AlphaDropout(1.0 - float(cfg.get("rate", 0.5))), layerName=name), "layer"
    if cls == "GaussianDropout":
        return nn.DropoutLayer(nn.GaussianDropout(float(cfg.get("rate", 0.5))), layerName=name), "layer"
    if cls == "GaussianNoise":
        return nn.DropoutLayer(nn.GaussianNoise(float(cfg.get("stddev", 0.1))), layerName=name), "layer"
    if cls == "Activation":
        return nn.ActivationLayer(_act(cfg), layerName=name), "layer"
    if cls == "LeakyReLU":
        return nn.ActivationLayer(nn.activations.ActivationLReLU(alpha=float(cfg.get("alpha", cfg.get("negative_slope", 0.3)))), layerName=name), "layer"
    if cls == "ReLU":
        return nn.ActivationLayer("RELU", layerName=name), "layer"
    if cls == "Softmax":
        return nn.ActivationLayer("SOFTMAX", layerName=name), "layer"
    if cls == "BatchNormalization":
        return nn.BatchNormalization(eps=float(cfg.get("epsilon", 1e-3)), decay=float(cfg.get("momentum", 0.99)), layerName=name), "layer"
    if cls == "Embedding":
        return nn.EmbeddingSequenceLayer(nIn=cfg["input_dim"], nOut=cfg["output_dim"], hasBias=False, activation="IDENTITY", layerName=name), "layer"
    if cls == "LSTM":
        l = nn.LSTM(nOut=cfg["units"], activation=_act(cfg), gateActivationFn=_ACT.get(cfg.get("recurrent_activation", "sigmoid"), "SIGMOID"), layerName=name)
        return (l if cfg.get("return_sequences", False) else nn.LastTimeStep(l)), "layer"
    if cls == "SimpleRNN":
        l = nn.SimpleRnn(nOut=cfg["units"], activation=_act(cfg), layerName=name)
        return (l if cfg.get("return_sequences", False) else nn.LastTimeStep(l)), "layer"
    if cls == "ZeroPadding2D":
        p = cfg.get("padding", 1)
        p = [p, p, p, p] if isinstance(p, int) else ([p[0], p[0], p[1], p[1]] if isinstance(p[0], int) else [p[0][0], p[0][1], p[1][0], p[1][1]])
        return nn.ZeroPaddingLayer(*[int(v) for v in p], layerName=name), "layer"
    if cls == "Cropping2D":
        p = cfg.get("cropping", 0)
        p = [p, p, p, p] if isinstance(p, int) else ([p[0], p[0], p[1], p[1]] if isinstance(p[0], int) else [p[0][0], p[0][1], p[1][0], p[1][1]])
        return nn.Cropping2D(*[int(v) for v in p], layerName=name), "layer"
    if cls == "UpSampling2D":
        return nn.Upsampling2D(_pair(cfg.get("size", 2)), layerName=name), "layer"
    if cls in ("Conv3D", "Convolution3D"):
        return nn.Convolution3D(kernelSize=_triple(cfg["kernel_size"]), stride=_triple(cfg.get("strides", 1)), nOut=cfg["filters"], activation=_act(cfg),
                                convolutionMode=_mode(cfg), dilation=_triple(cfg.get("dilation_rate", 1)), hasBias=cfg.get("use_bias", True), layerName=name), "layer"
    if cls in ("Conv3DTranspose", "Deconvolution3D"):
        return nn.Deconvolution3D(kernelSize=_triple(cfg["kernel_size"]), stride=_triple(cfg.get("strides", 1)), nOut=cfg["filters"], activation=_act(cfg),
                                  convolutionMode=_mode(cfg), hasBias=cfg.get("use_bias", True), layerName=name), "layer"
    if cls in ("MaxPooling3D", "AveragePooling3D"):
        ps = _triple(cfg.get("pool_size", 2))
        return nn.Subsampling3DLayer("MAX" if cls.startswith("Max") else "AVG", kernelSize=ps, stride=_triple(cfg.get("strides") or ps), convolutionMode=_mode(cfg),
                                     layerName=name), "layer"
    if cls in ("GlobalAveragePooling3D", "GlobalMaxPooling3D"):
        return nn.GlobalPoolingLayer("AVG" if "Average" in cls else "MAX", layerName=name), "layer"
    if cls in ("AtrousConvolution2D", "AtrousConv2D"):                                        # Keras 1: the dilation is called atrous_rate
        return nn.ConvolutionLayer([cfg["nb_row"], cfg["nb_col"]], _pair(cfg.get("subsample", 1)), nOut=cfg["nb_filter"], activation=_act(cfg),
                                   convolutionMode="Same" if cfg.get("border_mode") == "same" else "Truncate", dilation=_pair(cfg.get("atrous_rate", 1)),
                                   hasBias=cfg.get("bias", True), layerName=name), "layer"
    if cls == "ZeroPadding1D":
        p = cfg.get("padding", 1)
        return nn.ZeroPadding1DLayer(*([int(p)] * 2 if isinstance(p, int) else [int(v) for v in p]), layerName=name), "layer"
    if cls == "ZeroPadding3D":
        return nn.ZeroPadding3DLayer(*_sides(cfg.get("padding", 1), 3), layerName=name), "layer"
    if cls == "Cropping1D":
        p = cfg.get("cropping", 1)
        return nn.Cropping1D(*([int(p)] * 2 if isinstance(p, int) else [int(v) for v in p]), layerName=name), "layer"
    if cls == "Cropping3D":
        return nn.Cropping3D(*_sides(cfg.get("cropping", 1), 3), layerName=name), "layer"
    if cls == "UpSampling1D":
        sz = cfg.get("size", 2)
        return nn.Upsampling1D(int(sz[0] if isinstance(sz, (list, tuple)) else sz), layerName=name), "layer"
    if cls == "UpSampling3D":
        return nn.Upsampling3D(_triple(cfg.get("size", 2)), layerName=name), "layer"
    if cls == "SpaceToDepth":
        return nn.SpaceToDepthLayer(int(cfg.get("block_size", 2)), layerName=name), "layer"
    if cls in ("LRN", "LRN2D"):
        return nn.LocalResponseNormalization(n=float(cfg.get("n", 5)), k=float(cfg.get("k", 2)), alpha=float(cfg.get("alpha", 1e-4)), beta=float(cfg.get("beta", 0.75)),
                                             layerName=name), "layer"
    if cls == "PoolHelper":
        from ..nn.conf.graphconf import PoolHelperVertex
        return PoolHelperVertex(), "vertex"
    if cls == "PReLU":
        shared = cfg.get("shared_axes")
        return nn.PReLULayer(layerName=name, sharedAxesChannelsLast=[int(a) for a in shared] if shared else None), "layer"
    if cls == "ELU":
        return nn.ActivationLayer(nn.activations.ActivationELU(alpha=float(cfg.get("alpha", 1.0))), layerName=name), "layer"
    if cls == "ThresholdedReLU":
        return nn.ActivationLayer(nn.activations.ActivationThresholdedReLU(theta=float(cfg.get("theta", 1.0))), layerName=name), "layer"
    if cls == "RepeatVector":
        return nn.RepeatVector(int(cfg["n"]), layerName=name), "layer"
    if cls == "Reshape":
        return ReshapePreprocessor(cfg["target_shape"]), "preprocessor"
    if cls == "Permute":
        return PermutePreprocessor(cfg["dims"]), "preprocessor"
    if cls == "Masking":
        return float(cfg.get("mask_value", 0.0)), "masking"
    if cls == "Bidirectional":
        inner = cfg["layer"]
        icfg = dict(inner["config"])
        seq = icfg.get("return_sequences", False)
        icfg["return_sequences"] = True
        l, _ = _map_layer(inner["class_name"], icfg, False, None)
        mode = {"concat": "CONCAT", "sum": "ADD", "mul": "MUL", "ave": "AVERAGE"}.get(cfg.get("merge_mode", "concat"))
        if mode is None:
            raise UnsupportedKerasConfigurationException(f"Unsupported Bidirectional merge mode {cfg.get('merge_mode')}")
        b = nn.Bidirectional(mode, l, layerName=name)
        return (b if seq else nn.LastTimeStep(b)), "layer"
    if cls == "TimeDistributed":
        inner = cfg["layer"]
        l, what = _map_layer(inner["class_name"], dict(inner["config"], name=name), is_last, loss)
        if what != "layer":
            raise UnsupportedKerasConfigurationException(f"TimeDistributed around {inner['class_name']}")
        if type(l).__name__ == "OutputLayer":                                             # a per-step output layer is the recurrent output layer
            return nn.RnnOutputLayer(loss, nOut=l.nOut, activation=_act(inner["config"]), hasBias=l.hasBias, layerName=name), "layer"
        return nn.TimeDistributed(l, layerName=name), "layer"
    if cls == "LocallyConnected2D":
        return nn.LocallyConnected2D(nOut=cfg["filters"], kernel=_pair(cfg["kernel_size"]), stride=_pair(cfg.get("strides", 1)), activation=_act(cfg),
                                     convolutionMode=_mode(cfg), hasBias=cfg.get("use_bias", True), layerName=name), "layer"
    if cls == "LocallyConnected1D":
        k = cfg["kernel_size"]
        st = cfg.get("strides", 1)
        return nn.LocallyConnected1D(nOut=cfg["filters"], kernel=int(k[0] if isinstance(k, (list, tuple)) else k), stride=int(st[0] if isinstance(st, (list, tuple)) else st),
                                     activation=_act(cfg), convolutionMode=_mode(cfg), hasBias=cfg.get("use_bias", True), layerName=name), "layer"
    if cls == "Lambda":
        if name not in _LAMBDA_LAYERS:
            raise UnsupportedKerasConfigurationException(f"No SameDiff Lambda layer found for Lambda layer {name}. You can register a SameDiff Lambda layer using "
                                                         f"KerasLayer.registerLambdaLayer(lambdaLayerName, sameDiffLambdaLayer)")
        return _LAMBDA_LAYERS[name], "layer"
    if cls in _CUSTOM_LAYERS:
        return _CUSTOM_LAYERS[cls](cfg), "layer"
    if cls == "Attention":
        if cfg.get("score_mode", "dot") != "dot":
            raise InvalidKerasConfigurationException(f"Invalid score mode {cfg.get('score_mode')}")
        from ..nn.conf.graphconf import DotProductAttentionVertex
        v = DotProductAttentionVertex(scaleFactor=1.0, dropoutProbability=float(cfg.get("dropout", 0.0)), useCausalMask=bool(cfg.get("causal", False)))
        v._keras_use_scale = bool(cfg.get("use_scale", False))          # the learned scalar arrives with the weights
        return v, "attention"
    if cls == "Add":
        return ElementWiseVertex("Add"), "vertex"
    if cls == "Multiply":
        return ElementWiseVertex("Product"), "vertex"
    if cls == "Subtract":
        return ElementWiseVertex("Subtract"), "vertex"
    if cls == "Average":
        return ElementWiseVertex("Average"), "vertex"
    if cls == "Maximum":
        return ElementWiseVertex("Max"), "vertex"
    if cls == "Concatenate":
        return MergeVertex(), "vertex"
    raise UnsupportedKerasConfigurationException(f"Unsupported keras layer type {cls}")


def _input_type(shape):
    shape = [s for s in shape[1:]]
    if len(shape) == 4:
        return nn.InputType.convolutional3D(shape[0], shape[1], shape[2], shape[3]), "cnn3d"   # NDHWC -> d, h, w, c
    if len(shape) == 3:
        return nn.InputType.convolutional(shape[0], shape[1], shape[2]), "cnn"           # NHWC -> h, w, c
    if len(shape) == 2:
        return nn.InputType.recurrent(shape[1], shape[0] if shape[0] else -1), "rnn"
    return nn.InputType.feedForward(shape[0]), "ff"


def _convert_weights(layer, arrays, flatten_from=None):
    """Keras arrays -> {param name: tensor} for a DL4J layer."""
    t = [torch.from_numpy(np.asarray(a, dtype=np.float32)) for a in arrays]
    cls = type(layer).__name__
    if cls in ("LastTimeStep", "MaskZeroLayer", "TimeDistributed"):
        return _convert_weights(layer.underlying, arrays)
    if cls == "Bidirectional":
        half = len(arrays) // 2                                                        # forward copy's arrays, then the backward copy's
        out = {"f" + k: v for k, v in _convert_weights(layer.fwd, arrays[:half]).items()}
        out.update({"b" + k: v for k, v in _convert_weights(layer.bwd, arrays[half:]).items()})
        return out
    if cls == "RnnOutputLayer":
        out = {"W": t[0]}
        if len(t) > 1:
            out["b"] = t[1].reshape(1, -1)
        return out
    if cls == "Convolution3D":
        out = {"W": t[0].permute(4, 3, 0, 1, 2)}                                       # DHWIO -> OIDHW
        if len(t) > 1:
            out["b"] = t[1].reshape(1, -1)
        return out
    if cls == "Deconvolution3D":
        out = {"W": t[0].permute(4, 3, 0, 1, 2)}                                       # [kd, kh, kw, out, in] -> [in, out, kd, kh, kw]
        if len(t) > 1:
            out["b"] = t[1].reshape(1, -1)
        return out
    if cls == "PReLULayer":
        a = t[0]
        return {"W": a.permute(a.dim() - 1, *range(a.dim() - 1)) if a.dim() > 1 else a}   # channels last -> channels first
    if cls == "LocallyConnected2D":
        kh, kw = layer.kernel
        W = t[0]                                                                       # [positions, kh*kw*in, out], features in (kh, kw, in) order
        W = W.reshape(W.shape[0], kh, kw, -1, W.shape[-1]).permute(0, 3, 1, 2, 4).reshape(W.shape[0], -1, W.shape[-1])
        out = {"W": W}
        if len(t) > 1:
            if t[1].numel() != layer.nOut:
                raise UnsupportedKerasConfigurationException("LocallyConnected2D with one bias per output position (the layer here shares the bias over positions)")
            out["b"] = t[1].reshape(1, -1)
        return out
    if cls == "LocallyConnected1D":
        k = layer.kernel
        W = t[0]                                                                       # [steps, k*in, out], features in (k, in) order
        W = W.reshape(W.shape[0], k, -1, W.shape[-1]).permute(0, 2, 1, 3).reshape(W.shape[0], -1, W.shape[-1])
        out = {"W": W}
        if len(t) > 1:
            if t[1].numel() != layer.nOut:
                raise UnsupportedKerasConfigurationException("LocallyConnected1D with one bias per output step (the layer here shares the bias over steps)")
            out["b"] = t[1].reshape(1, -1)
        return out
    if cls in ("DenseLayer", "OutputLayer"):
        W = t[0]
        if flatten_from is not None:                                                   # rows are in (h, w, c) order; DL4J flattens (c, h, w)
            dims = list(flatten_from)                                                  # spatial extents ..., channels
            n = len(dims)
            W = W.reshape(*dims, -1).permute(n - 1, *range(n - 1), n).reshape(int(np.prod(dims)), -1)
        out = {"W": W}
        if len(t) > 1:
            out["b"] = t[1].reshape(1, -1)
        return out
    if cls == "ConvolutionLayer":
        out = {"W": t[0].permute(3, 2, 0, 1)}                                          # HWIO -> OIHW
        if len(t) > 1:
            out["b"] = t[1].reshape(1, -1)
        return out
    if cls == "Deconvolution2D":
        out = {"W": t[0].permute(3, 2, 0, 1)}                                          # [kh, kw, out, in] -> [in, out, kh, kw]
        if len(t) > 1:
            out["b"] = t[1].reshape(1, -1)
        return out
    if cls == "Convolution1DLayer":
        out = {"W": t[0].permute(2, 1, 0).unsqueeze(-1)}                               # [k, in, out] -> [out, in, k, 1]
        if len(t) > 1:
            out["b"] = t[1].reshape(1, -1)
        return out
    if cls == "DepthwiseConvolution2D":
        out = {"W": t[0].permute(3, 2, 0, 1)}                                          # [kh, kw, in, mult] -> [mult, in, kh, kw]
        if len(t) > 1:
            out["b"] = t[1].reshape(1, -1)
        return out
    if cls == "SeparableConvolution2D":
        out = {"W": t[0].permute(3, 2, 0, 1), "pW": t[1].permute(3, 2, 0, 1)}
        if len(t) > 2:
            out["b"] = t[2].reshape(1, -1)
        return out
    if cls == "BatchNormalization":
        gamma, beta, mean, var = t if len(t) == 4 else (torch.ones_like(t[0]), *t)
        return {"gamma": gamma.reshape(1, -1), "beta": beta.reshape(1, -1), "mean": mean.reshape(1, -1), "var": var.reshape(1, -1)}
    if cls == "EmbeddingSequenceLayer":
        return {"W": t[0]}
    if cls == "LSTM":
        # Keras gate order (i, f, c, o) -> DL4J column blocks (c, f, o, i)
        def reorder(m):
            i, f, c, o = m.chunk(4, dim=-1)
            return torch.cat([c, f, o, i], dim=-1)
        out = {"W": reorder(t[0]), "RW": reorder(t[1])}
        if len(t) > 2:
            out["b"] = reorder(t[2]).reshape(1, -1)
        return out
    if cls == "SimpleRnn":
        out = {"W": t[0], "RW": t[1]}
        if len(t) > 2:
            out["b"] = t[2].reshape(1, -1)
        return out
    return {}


def _set_params(net, key, layer, arrays, flatten_from=None):
    table = net.paramTable()
    conv = _convert_weights(layer, arrays, flatten_from)
    with torch.no_grad():
        for pn, val in conv.items():
            k = f"{key}_{pn}"
            if pn == "var" and k not in table:
                k2 = f"{key}_log10stdev"
                if k2 in table:
                    dst = table[k2].t
                    dst.copy_((0.5 * torch.log10(val.clamp_min(1e-30))).reshape(dst.shape))     # stored as log10(stdev)
                    continue
            if k not in table:
                continue
            dst = table[k].t
            if tuple(dst.shape) != tuple(val.shape):
                if dst.numel() != val.numel():
                    raise InvalidKerasConfigurationException(f"weight shape mismatch for {k}: keras {tuple(val.shape)} vs {tuple(dst.shape)}")
                val = val.reshape(dst.shape)
            dst.copy_(val)
    if getattr(net, "flat_shadow", None) is not None:
        net._refresh_shadow()


def _load_weights(weights):
    if weights is None:
        return {}
    if isinstance(weights, dict):
        return {k: list(v) for k, v in weights.items()}
    path = str(weights)
    if path.endswith(".npz"):
        z = np.load(path)
        out = {}
        for k in sorted(z.files, key=lambda s: (s.rsplit("/", 1)[0], int(s.rsplit("/", 1)[1]))):
            out.setdefault(k.rsplit("/", 1)[0], []).append(z[k])
        return out
    # HDF5: the importer's own reader (importers/hdf5.py) - Keras stores, under /model_weights (or at the root of a weights-only
    # file), one group per layer with a weight_names attribute listing its datasets
    from .hdf5 import Hdf5Archive
    out = {}
    with Hdf5Archive(path) as ar:
        root = ("model_weights",) if "model_weights" in ar.getGroups() else ()
        layer_names = ar.readAttributeAsStringList("layer_names", *root) or ar.getGroups(*root)
        for lname in layer_names:
            names = ar.readAttributeAsStringList("weight_names", *root, lname)
            out[lname] = [ar.readDataSet(n, *root, lname) for n in names]
    return out


def _is_hdf5(path):
    try:
        with open(path, "rb") as f:
            return f.read(8) == b"\x89HDF\r\n\x1a\n"
    except (OSError, TypeError, ValueError):
        return False


class KerasModelImport:
    @staticmethod
    def _config(model_json):
        if isinstance(model_json, str) and model_json.lstrip().startswith("{"):
            cfg = json.loads(model_json)
        elif _is_hdf5(model_json):
            # a full-model .h5 file: architecture and training configuration are JSON attributes of the root group
            from .hdf5 import Hdf5Archive
            with Hdf5Archive(model_json) as ar:
                if not ar.hasAttribute("model_config"):
                    raise InvalidKerasConfigurationException("the HDF5 file has no model_config attribute (a weights-only file: pass the "
                                                             "architecture JSON as the first argument and this file as weights)")
                cfg = ar.readAttributeAsJson("model_config")
                if ar.hasAttribute("training_config") and "training_config" not in cfg:
                    cfg["training_config"] = ar.readAttributeAsJson("training_config")
        else:
            cfg = json.load(open(model_json))
        loss = None
        tc = cfg.get("training_config") or {}
        l = tc.get("loss")
        if isinstance(l, dict):
            l = l.get("class_name") or next(iter(l.values()), None)
        if isinstance(l, str):
            key = "".join("_" + c.lower() if c.isupper() else c for c in l).lstrip("_") if any(c.isupper() for c in l) else l
            loss = _LOSS.get(key) or _LOSS.get(l)
        return cfg, loss

    @staticmethod
    def importKerasSequentialModelAndWeights(model_json, weights=None, enforceTrainingConfig=False, loss=None):
        cfg, cfg_loss = KerasModelImport._config(model_json)
        loss = loss or cfg_loss
        if cfg.get("class_name") != "Sequential":
            raise InvalidKerasConfigurationException(f"Model class name must be Sequential (found {cfg.get('class_name')})")
        layers_cfg = cfg["config"]["layers"] if isinstance(cfg["config"], dict) else cfg["config"]
        in_shape = None
        for lc in layers_cfg:
            c = lc["config"]
            in_shape = c.get("batch_input_shape") or c.get("batch_shape") or in_shape
            if in_shape:
                break
        if in_shape is None:
            raise InvalidKerasConfigurationException("could not determine the input shape (no batch_input_shape on the first layer)")
        it, kind = _input_type(in_shape)
        lb = nn.NeuralNetConfiguration.Builder().list()
        mapped = []                      # (dl4j index, keras name, layer, flatten_from)
        idx, cur, pending_flatten = 0, it, None
        pending_pp, pending_mask = [], None
        real = [lc for lc in layers_cfg if lc["class_name"] != "InputLayer"]
        for k, lc in enumerate(real):
            layer, what = _map_layer(lc["class_name"], lc["config"], k == len(real) - 1, loss)
            if what == "flatten":
                if cur.kind == nn.InputType.CNN:
                    pending_flatten = (cur.height, cur.width, cur.channels)
                elif cur.kind == nn.InputType.CNN3D:
                    pending_flatten = (cur.depth, cur.height, cur.width, cur.channels)
                elif cur.kind == nn.InputType.RNN and cur.timeSeriesLength and cur.timeSeriesLength > 0:
                    pending_flatten = (cur.timeSeriesLength, cur.size)
                continue
            if what in ("input", "skip"):
                continue
            if what in ("vertex", "attention"):
                raise InvalidKerasConfigurationException("merge layers need the functional API: use importKerasModelAndWeights")
            if what == "masking":
                pending_mask = layer
                continue
            if what == "preprocessor":
                pending_pp.append(layer)
                cur = layer.output_type(cur)
                if k == len(real) - 1:                                                 # nothing follows to carry it: an identity layer does
                    layer, what = nn.ActivationLayer("IDENTITY", layerName=lc["config"].get("name")), "layer"
                else:
                    continue
            if pending_mask is not None and (getattr(layer, "IS_RECURRENT", False) or type(layer).__name__ == "LastTimeStep"):
                layer = nn.MaskZeroLayer(underlying=layer, maskingValue=pending_mask, layerName=lc["config"].get("name"))
                pending_mask = None
            if pending_pp:
                auto = layer.preprocessor_for(cur)
                lb.inputPreProcessor(idx, ComposableInputPreProcessor(pending_pp + ([auto] if auto is not None else [])) if (auto is not None or len(pending_pp) > 1) else pending_pp[0])
                if auto is not None:
                    cur = auto.output_type(cur)
                pending_pp = []
                lb.layer(idx, layer)
                mapped.append((idx, lc["config"]["name"], layer, None))
                layer.setNIn(cur, True)
                cur = layer.output_type(cur)
                idx += 1
                continue
            lb.layer(idx, layer)
            mapped.append((idx, lc["config"]["name"], layer, pending_flatten if type(layer).__name__ in ("DenseLayer", "OutputLayer") else None))
            if pending_flatten is not None and type(layer).__name__ in ("DenseLayer", "OutputLayer"):
                pending_flatten = None
            pp = layer.preprocessor_for(cur)
            if pp is not None:
                cur = pp.output_type(cur)
            layer.setNIn(cur, True)
            cur = layer.output_type(cur)
            idx += 1
        lb.setInputType(it).validateOutputLayerConfig(False)
        net = nn.MultiLayerNetwork(lb.build()).init()
        if weights is None and not (isinstance(model_json, str) and model_json.lstrip().startswith("{")) and _is_hdf5(model_json):
            weights = model_json                      # full-model file: the weights sit beside the configuration
        w = _load_weights(weights)
        for i, kname, layer, ff in mapped:
            if kname in w and w[kname]:
                _set_params(net, str(i), net.conf.layers()[i], w[kname], ff)
        net.kerasInputLayout = {"cnn": "NHWC", "cnn3d": "NDHWC", "rnn": "NWC"}.get(kind, "NC")
        return net

    @staticmethod
    def importKerasModelAndWeights(model_json, weights=None, enforceTrainingConfig=False, loss=None):
        cfg, cfg_loss = KerasModelImport._config(model_json)
        loss = loss or cfg_loss
        if cfg.get("class_name") == "Sequential":
            return KerasModelImport.importKerasSequentialModelAndWeights(model_json, weights, enforceTrainingConfig, loss)
        c = cfg["config"]
        gb = nn.NeuralNetConfiguration.Builder().graphBuilder()
        names = lambda spec: [s[0] for s in spec]
        in_names = names(c["input_layers"])
        out_names = names(c["output_layers"])
        gb.addInputs(*in_names)
        its, mapped, flatten_of = [], [], {}
        by_name = {lc["config"]["name"] if "name" in lc["config"] else lc["name"]: lc for lc in c["layers"]}
        for n in in_names:
            sh = by_name[n]["config"].get("batch_input_shape") or by_name[n]["config"].get("batch_shape")
            its.append(_input_type(sh)[0])
        gb.setInputTypes(*its)
        alias, mask_of, scaled = {}, {}, []
        for lc in c["layers"]:
            name = lc.get("name") or lc["config"]["name"]
            if lc["class_name"] == "InputLayer":
                continue
            inbound = lc.get("inbound_nodes") or []
            srcs = []
            if inbound:
                node0 = inbound[0]
                if isinstance(node0, dict):                                            # Keras 3 format
                    def walk(o):
                        if isinstance(o, dict) and o.get("class_name") == "__keras_tensor__":
                            srcs.append(o["config"]["keras_history"][0])
                        elif isinstance(o, dict):
                            [walk(v) for v in o.values()]
                        elif isinstance(o, (list, tuple)):
                            [walk(v) for v in o]
                    walk(node0.get("args", []))
                else:
                    srcs = [s[0] for s in node0]
            srcs = [alias.get(s, s) for s in srcs]
            layer, what = _map_layer(lc["class_name"], lc["config"], name in out_names, loss)
            if what == "flatten":
                alias[name] = srcs[0]
                flatten_of[name] = srcs[0]
                continue
            if what == "masking":
                alias[name] = srcs[0]
                mask_of[name] = layer
                continue
            if what == "preprocessor":
                gb.addVertex(name, PreprocessorVertex(layer), *srcs)
                continue
            raw = [s[0] for s in inbound[0]] if inbound and not isinstance(inbound[0], dict) else []
            masked = [mask_of[r] for r in raw if r in mask_of]
            if masked and what == "layer" and (getattr(layer, "IS_RECURRENT", False) or type(layer).__name__ == "LastTimeStep"):
                layer = nn.MaskZeroLayer(underlying=layer, maskingValue=masked[0], layerName=name)
            if what == "attention":
                if len(srcs) == 3:
                    srcs = [srcs[0], srcs[2], srcs[1]]                                 # Keras passes [query, value, key]
                gb.addVertex(name, layer, *srcs)
                scaled.append((name, layer))
                continue
            if what == "vertex":
                gb.addVertex(name, layer, *srcs)
            else:
                gb.addLayer(name, layer, *srcs)
                mapped.append((name, layer, srcs))
        gb.setOutputs(*[alias.get(o, o) for o in out_names]).validateOutputLayerConfig(False)
        types = gb.getLayerActivationTypes()
        conf = gb.build()
        from ..nn.graph import ComputationGraph
        net = ComputationGraph(conf).init()
        if weights is None and not (isinstance(model_json, str) and model_json.lstrip().startswith("{")) and _is_hdf5(model_json):
            weights = model_json                      # full-model file: the weights sit beside the configuration
        w = _load_weights(weights)
        for name, vertex in scaled:
            if vertex._keras_use_scale and w.get(name):
                vertex.scaleFactor = float(np.asarray(w[name][0]).reshape(-1)[0])
        for name, layer, srcs in mapped:
            if name in w and w[name]:
                ff = None
                src_t = types.get(srcs[0]) if srcs else None
                if type(layer).__name__ in ("DenseLayer", "OutputLayer") and src_t is not None and src_t.kind == nn.InputType.CNN:
                    ff = (src_t.height, src_t.width, src_t.channels)
                elif type(layer).__name__ in ("DenseLayer", "OutputLayer") and src_t is not None and src_t.kind == nn.InputType.CNN3D:
                    ff = (src_t.depth, src_t.height, src_t.width, src_t.channels)
                _set_params(net, name, conf.vertices[name].layer, w[name], ff)
        return net

    @staticmethod
    def registerLambdaLayer(lambdaLayerName, sameDiffLambdaLayer):
        """``KerasLayer.registerLambdaLayer``: the layer that stands for the Keras ``Lambda`` layer of that name."""
        _LAMBDA_LAYERS[lambdaLayerName] = sameDiffLambdaLayer

    @staticmethod
    def clearLambdaLayers():
        _LAMBDA_LAYERS.clear()

    @staticmethod
    def registerCustomLayer(layerName, factory):
        """``KerasLayer.registerCustomLayer``: ``factory(keras config dict) -> layer`` for a Keras class this importer does not know."""
        _CUSTOM_LAYERS[layerName] = factory

    @staticmethod
    def importKerasModelConfiguration(model_json):
        return KerasModelImport.importKerasModelAndWeights(model_json).conf

    @staticmethod
    def importKerasSequentialConfiguration(model_json):
        return KerasModelImport.importKerasSequentialModelAndWeights(model_json).conf
