"""Updater ops (``headers/updaters.h``): each returns (update, new state...) like the native ops in
``libnd4j/include/ops/declarable/generic/updaters/*.cpp`` and shares its math with ``nn.updaters``."""
from __future__ import annotations

import torch

from ..nn import updaters as U
from .registry import op


def _run(cfg, g, states, lr, t):
    g = g.clone()
    st = torch.cat([s.reshape(-1).clone() for s in states]) if states else g.new_zeros(0)
    if isinstance(cfg, U.Nesterovs):
        cfg.apply(g, st.view_as(g), lr, t)
    else:
        cfg.apply(g, st, lr, t)
    n = g.numel()
    return (g,) + tuple(st[i * n:(i + 1) * n].view_as(g) for i in range(len(states)))


op("sgd_updater")(lambda g, lr=1e-3, **kw: g * lr)
op("nesterovs_updater", n_out=2)(lambda g, v, lr=0.1, momentum=0.9, **kw: _run(U.Nesterovs(lr, momentum), g, [v], lr, 0))
op("adam_updater", n_out=3)(lambda g, v, m, lr=1e-3, beta1=0.9, beta2=0.999, epsilon=1e-8, iteration=0, **kw:
                            (lambda r: (r[0], r[2], r[1]))(_run(U.Adam(lr, beta1, beta2, epsilon), g, [m, v], lr, int(iteration))))
op("ada_max_updater", n_out=3)(lambda g, u, m, lr=1e-3, beta1=0.9, beta2=0.999, epsilon=1e-8, iteration=0, **kw:
                               (lambda r: (r[0], r[2], r[1]))(_run(U.AdaMax(lr, beta1, beta2, epsilon), g, [m, u], lr, int(iteration))))
op("nadam_updater", n_out=3)(lambda g, v, m, lr=1e-3, beta1=0.9, beta2=0.999, epsilon=1e-8, iteration=0, **kw:
                             (lambda r: (r[0], r[2], r[1]))(_run(U.Nadam(lr, beta1, beta2, epsilon), g, [m, v], lr, int(iteration))))
op("ams_grad_updater", n_out=4)(lambda g, v, m, h, lr=1e-3, beta1=0.9, beta2=0.999, epsilon=1e-8, iteration=0, **kw:
                                (lambda r: (r[0], r[2], r[1], r[3]))(_run(U.AMSGrad(lr, beta1, beta2, epsilon), g, [m, v, h], lr, int(iteration))))
op("adabelief_updater", n_out=3)(lambda g, u, m, lr=1e-3, beta1=0.9, beta2=0.999, epsilon=1e-14, iteration=0, **kw:
                                 (lambda r: (r[0], r[2], r[1]))(_run(U.AdaBelief(lr, beta1, beta2, epsilon), g, [m, u], lr, int(iteration))))
op("ada_grad_updater", n_out=2)(lambda g, h, lr=0.1, epsilon=1e-6, **kw: _run(U.AdaGrad(lr, epsilon), g, [h], lr, 0))
op("rms_prop_updater", n_out=2)(lambda g, s, lr=0.1, rmsDecay=0.95, epsilon=1e-8, **kw: _run(U.RmsProp(lr, rmsDecay, epsilon), g, [s], lr, 0))
op("ada_delta_updater", n_out=3)(lambda g, msg, msdx, rho=0.95, epsilon=1e-6, **kw: _run(U.AdaDelta(rho, epsilon), g, [msg, msdx], 0.0, 0))
