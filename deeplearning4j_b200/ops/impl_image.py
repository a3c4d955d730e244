"""Image ops (``headers/images.h`` + image entries of ``headers/parity_ops.h``): colour-space
conversions, resizes, crop_and_resize, non-max suppression, bounding boxes, hue/saturation/contrast.
Images are NHWC (channels last) unless ``dimC`` says otherwise, as in the native ops."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .registry import op


def _cl(x, dimC):
    d = int(dimC) % x.dim()
    return x.movedim(d, -1), d


def _mat(x, m, dimC=-1):
    xc, d = _cl(x, dimC)
    M = torch.tensor(m, dtype=x.dtype, device=x.device)
    return (xc @ M.t()).movedim(-1, d)


_YUV = [[0.299, 0.587, 0.114], [-0.14714119, -0.28886916, 0.43601035], [0.61497538, -0.51496512, -0.10001026]]
_YIQ = [[0.299, 0.587, 0.114], [0.59590059, -0.27455667, -0.32134392], [0.21153661, -0.52273617, 0.31119955]]
op("rgb_to_yuv")(lambda x, dimC=-1, **kw: _mat(x, _YUV, dimC))
op("yuv_to_rgb")(lambda x, dimC=-1, **kw: _mat(x, torch.linalg.inv(torch.tensor(_YUV)).tolist(), dimC))
op("rgb_to_yiq")(lambda x, dimC=-1, **kw: _mat(x, _YIQ, dimC))
op("yiq_to_rgb")(lambda x, dimC=-1, **kw: _mat(x, torch.linalg.inv(torch.tensor(_YIQ)).tolist(), dimC))
op("rgb_to_grs")(lambda x, dimC=-1, **kw: (_cl(x, dimC)[0] * torch.tensor([0.2989, 0.5870, 0.1140], dtype=x.dtype, device=x.device)).sum(-1, keepdim=True).movedim(-1, int(dimC) % x.dim()))


@op("rgb_to_hsv")
def rgb_to_hsv(x, dimC=-1, **kw):
    xc, d = _cl(x, dimC)
    r, g, b = xc.unbind(-1)
    mx, mn = xc.amax(-1), xc.amin(-1)
    delta = mx - mn
    h = torch.zeros_like(mx)
    nz = delta > 0
    h = torch.where(nz & (mx == r), ((g - b) / delta.clamp_min(1e-30)) % 6, h)
    h = torch.where(nz & (mx == g) & (mx != r), (b - r) / delta.clamp_min(1e-30) + 2, h)
    h = torch.where(nz & (mx == b) & (mx != r) & (mx != g), (r - g) / delta.clamp_min(1e-30) + 4, h)
    h = h / 6.0
    s = torch.where(mx > 0, delta / mx.clamp_min(1e-30), torch.zeros_like(mx))
    return torch.stack([h, s, mx], -1).movedim(-1, d)


@op("hsv_to_rgb")
def hsv_to_rgb(x, dimC=-1, **kw):
    xc, d = _cl(x, dimC)
    h, s, v = xc.unbind(-1)
    h6 = h * 6.0
    c = v * s
    xx = c * (1 - ((h6 % 2) - 1).abs())
    m = v - c
    z = torch.zeros_like(c)
    sel = h6.floor().long() % 6
    r = torch.stack([c, xx, z, z, xx, c], -1).gather(-1, sel.unsqueeze(-1)).squeeze(-1)
    g = torch.stack([xx, c, c, xx, z, z], -1).gather(-1, sel.unsqueeze(-1)).squeeze(-1)
    b = torch.stack([z, z, xx, c, c, xx], -1).gather(-1, sel.unsqueeze(-1)).squeeze(-1)
    return torch.stack([r + m, g + m, b + m], -1).movedim(-1, d)


@op("adjust_hue")
def adjust_hue(x, delta=0.0, dimC=-1, **kw):
    d = float(delta.reshape(-1)[0]) if isinstance(delta, torch.Tensor) else delta
    hsv = rgb_to_hsv(x, dimC)
    hc, dd = _cl(hsv, dimC)
    hc = torch.cat([((hc[..., :1] + d) % 1.0), hc[..., 1:]], -1)
    return hsv_to_rgb(hc.movedim(-1, dd), dimC)


@op("adjust_saturation")
def adjust_saturation(x, factor=1.0, dimC=-1, **kw):
    f = float(factor.reshape(-1)[0]) if isinstance(factor, torch.Tensor) else factor
    hsv = rgb_to_hsv(x, dimC)
    hc, dd = _cl(hsv, dimC)
    hc = torch.cat([hc[..., :1], (hc[..., 1:2] * f).clamp(0, 1), hc[..., 2:]], -1)
    return hsv_to_rgb(hc.movedim(-1, dd), dimC)


@op("adjust_contrast", "adjust_contrast_v2")
def adjust_contrast(x, factor=1.0, **kw):
    f = float(factor.reshape(-1)[0]) if isinstance(factor, torch.Tensor) else factor
    mean = x.mean(dim=(-3, -2), keepdim=True)
    return (x - mean) * f + mean


def _resize(x, size, mode, align=False, half_pixel=False, antialias=False):
    h, w = (int(v) for v in (size.reshape(-1).tolist() if isinstance(size, torch.Tensor) else size))
    xc = x.permute(0, 3, 1, 2) if x.dim() == 4 else x.permute(2, 0, 1).unsqueeze(0)
    dt = xc.dtype
    xf = xc.float()
    if mode == "nearest":
        if half_pixel:
            y = F.interpolate(xf, (h, w), mode="nearest-exact")
        else:
            ih, iw = xc.shape[2:]
            ys = (torch.arange(h, device=x.device) * (ih / h)).floor().long().clamp(0, ih - 1)
            xs = (torch.arange(w, device=x.device) * (iw / w)).floor().long().clamp(0, iw - 1)
            y = xf[:, :, ys][:, :, :, xs]
    elif mode == "area":
        y = F.interpolate(xf, (h, w), mode="area")
    else:
        y = F.interpolate(xf, (h, w), mode=mode, align_corners=bool(align), antialias=antialias)
    y = y.to(dt) if mode == "nearest" else y
    return y.permute(0, 2, 3, 1) if x.dim() == 4 else y.squeeze(0).permute(1, 2, 0)


op("resize_bilinear")(lambda x, size=None, height=None, width=None, alignCorners=False, halfPixelCenters=False, **kw:
                      _resize(x, size if size is not None else (height, width), "bilinear", alignCorners))
op("resize_nearest_neighbor")(lambda x, size=None, height=None, width=None, alignCorners=False, halfPixelCenters=False, **kw:
                              _resize(x, size if size is not None else (height, width), "nearest", half_pixel=halfPixelCenters))
op("resize_bicubic")(lambda x, size=None, alignCorners=False, halfPixelCenters=False, **kw: _resize(x, size, "bicubic", alignCorners))
op("resize_area")(lambda x, size=None, alignCorners=False, **kw: _resize(x, size, "area"))


@op("image_resize", "resize_images")
def image_resize(x, size, method=0, preserveAspectRatio=False, antialias=False, **kw):
    mode = {0: "bilinear", 1: "nearest", 2: "bicubic", 3: "area"}.get(int(method), "bilinear")
    return _resize(x, size, mode, antialias=bool(antialias) and mode in ("bilinear", "bicubic"))


@op("crop_and_resize")
def crop_and_resize(image, boxes, boxIndices, cropSize, method=0, extrapolationVal=0.0, **kw):
    ch, cw = (int(v) for v in (cropSize.reshape(-1).tolist() if isinstance(cropSize, torch.Tensor) else cropSize))
    n, H, W, C = image.shape
    out = []
    for b, bi in zip(boxes.float(), boxIndices.long()):
        y1, x1, y2, x2 = b.tolist()
        ys = torch.linspace(y1, y2, ch, device=image.device) * 2 - 1 if ch > 1 else torch.tensor([(y1 + y2) - 1], device=image.device)
        xs = torch.linspace(x1, x2, cw, device=image.device) * 2 - 1 if cw > 1 else torch.tensor([(x1 + x2) - 1], device=image.device)
        gy, gx = torch.meshgrid(ys, xs, indexing="ij")
        grid = torch.stack([gx, gy], -1).unsqueeze(0)
        img = image[bi].permute(2, 0, 1).unsqueeze(0).float()
        samp = F.grid_sample(img, grid, mode="bilinear" if int(method) == 0 else "nearest", padding_mode="zeros", align_corners=True)
        oob = ((grid.abs() > 1).any(-1)).unsqueeze(1)
        samp = torch.where(oob, torch.full_like(samp, extrapolationVal), samp)
        out.append(samp.squeeze(0).permute(1, 2, 0))
    return torch.stack(out).to(image.dtype)


def _iou(boxes):
    y1, x1, y2, x2 = boxes.unbind(-1)
    ya, yb = torch.minimum(y1, y2), torch.maximum(y1, y2)
    xa, xb = torch.minimum(x1, x2), torch.maximum(x1, x2)
    area = (yb - ya) * (xb - xa)
    iy = (torch.minimum(yb[:, None], yb[None]) - torch.maximum(ya[:, None], ya[None])).clamp_min(0)
    ix = (torch.minimum(xb[:, None], xb[None]) - torch.maximum(xa[:, None], xa[None])).clamp_min(0)
    inter = iy * ix
    return inter / (area[:, None] + area[None] - inter).clamp_min(1e-30)


def _nms(overlaps, scores, max_out, thr, score_thr):
    order = torch.argsort(scores, descending=True).tolist()
    keep = []
    for i in order:
        if scores[i] < score_thr or len(keep) >= max_out:
            break
        if all(float(overlaps[i, j]) <= thr for j in keep):
            keep.append(i)
    return torch.tensor(keep, dtype=torch.int32, device=scores.device)


@op("non_max_suppression", "non_max_suppression_v3", differentiable=False)
def non_max_suppression(boxes, scores, maxOutputSize=None, iouThreshold=0.5, scoreThreshold=float("-inf"), maxOutSize=None, **kw):
    m = maxOutputSize if maxOutputSize is not None else maxOutSize
    m = int(m.reshape(-1)[0]) if isinstance(m, torch.Tensor) else int(m)
    return _nms(_iou(boxes.float()), scores.float(), m, float(iouThreshold), float(scoreThreshold))


@op("non_max_suppression_overlaps", differentiable=False)
def non_max_suppression_overlaps(overlaps, scores, maxOutputSize=None, overlapThreshold=0.5, scoreThreshold=float("-inf"), **kw):
    m = int(maxOutputSize.reshape(-1)[0]) if isinstance(maxOutputSize, torch.Tensor) else int(maxOutputSize)
    return _nms(overlaps.float(), scores.float(), m, float(overlapThreshold), float(scoreThreshold))


@op("draw_bounding_boxes")
def draw_bounding_boxes(images, boxes, colors, **kw):
    out = images.clone()
    n, H, W, C = images.shape
    for b in range(n):
        for k, bx in enumerate(boxes[b]):
            y1, x1, y2, x2 = bx.tolist()
            r1, r2 = int(round(y1 * (H - 1))), int(round(y2 * (H - 1)))
            c1, c2 = int(round(x1 * (W - 1))), int(round(x2 * (W - 1)))
            if r1 > r2 or c1 > c2 or r1 >= H or c1 >= W or r2 < 0 or c2 < 0:
                continue
            col = colors[k % colors.shape[0]].to(out.dtype)
            r1c, r2c, c1c, c2c = max(r1, 0), min(r2, H - 1), max(c1, 0), min(c2, W - 1)
            if r1 >= 0:
                out[b, r1, c1c:c2c + 1] = col
            if r2 < H:
                out[b, r2, c1c:c2c + 1] = col
            if c1 >= 0:
                out[b, r1c:r2c + 1, c1] = col
            if c2 < W:
                out[b, r1c:r2c + 1, c2] = col
    return out


@op("fake_quant_with_min_max_vars", "fake_quant_with_min_max_vars_per_channel")
def fake_quant(x, mn, mx, numBits=8, narrowed=False, **kw):
    qmin = 1.0 if narrowed else 0.0
    qmax = float(2 ** int(numBits) - 1)
    scale = (mx - mn) / (qmax - qmin)
    zp = qmin - mn / scale
    nudged_zp = torch.where(zp < qmin, torch.full_like(zp, qmin), torch.where(zp > qmax, torch.full_like(zp, qmax), torch.round(zp)))
    nmin = (qmin - nudged_zp) * scale
    nmax = (qmax - nudged_zp) * scale
    xc = torch.minimum(torch.maximum(x, nmin), nmax)
    return torch.floor((xc - nmin) / scale + 0.5) * scale + nmin
