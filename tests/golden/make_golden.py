"""Generates tests/golden/attention_golden.npz by running the REFERENCE itself.

Run where the reference checkout is available (its path in the EMBER_REFERENCE environment variable):

    make -C oracle ref && python tests/golden/make_golden.py

The reference's Python package is copied to a scratch directory under /tmp
together with the two CPython extension modules that ``make -C oracle ref``
compiled from the reference's unmodified C sources (CPU backend), imported as
``ember`` from there, and attention is composed from its public operators:

    forward : em.softmax((q @ kT) * scale [+ mask], axis=-1) @ v
    backward: dV = pT @ dO ; dP = dO @ vT ; delta = em.sum(dP * p, -1, keepdims)
              dS = (p * (dP - delta)) * scale ; dQ = dS @ k ; dK = dST @ q

Transposes of rank-4 tensors are done in NumPy because the reference's
transpose is 2-D only. Inputs come from the bit-reproducible generator in
``inputs.py`` (seeds: q = seed, k = seed+100, v = seed+200, dO = seed+300), so the
fixture file stores outputs only.
"""
import glob
import os
import shutil
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
# the reference checkout: $EMBER_REFERENCE, else a folder named "reference" beside this repository
REF = os.environ.get("EMBER_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(HERE))), "reference")
if not os.path.isdir(os.path.join(REF, "ember")):
    raise SystemExit("make_golden.py: set EMBER_REFERENCE to a checkout of the reference project")
sys.path.insert(0, HERE)
from inputs import normal  # noqa: E402

ROOT = os.path.dirname(os.path.dirname(HERE))

CASES = {
    # name: (B, H, Lq, Lk, D, causal, seed, with_backward)
    "c1_fwd_f32": (2, 4, 128, 128, 64, False, 1, False),  # the reference-runnable float32 configuration
    "c1_causal": (1, 2, 128, 128, 64, True, 2, True),
    "ragged_causal": (1, 2, 48, 80, 32, True, 3, True),
    "ragged_noncausal": (1, 3, 37, 129, 64, False, 4, True),
    "decode": (2, 2, 1, 300, 64, False, 5, False),
    "d128": (1, 1, 130, 130, 128, True, 6, True),
}


LINEAR_CASES = {
    # name: (m, k, n, seed, with_bias) -- the reference's own Linear layer (ember/nn/layers.py:9-56)
    "lin_small": (5, 7, 3, 11, True),
    "lin_tile": (128, 64, 256, 12, True),
    "lin_ragged": (130, 257, 66, 13, True),
    "lin_nobias": (96, 160, 72, 14, False),
}


SOFTMAX_CASES = {
    # name: (rows, cols, seed) -- em.softmax (ember/tensor/tensor.py:430-437) and the reference's
    # CrossEntropyLoss (ember/loss/losses.py:30-56) with one-hot targets at column (7 * row) % cols
    "sm_small": (4, 7, 21),
    "sm_ragged": (33, 130, 22),
    "sm_wide": (6, 5000, 23),
}


def import_reference():
    tmp = tempfile.mkdtemp(prefix="ember_ref_")
    shutil.copytree(os.path.join(REF, "ember"), os.path.join(tmp, "ember"))
    sos = glob.glob(os.path.join(ROOT, "oracle", "_ref", "ember", "_core", "*.so"))
    assert len(sos) == 2, "run `make -C oracle ref` first"
    for so in sos:
        shutil.copy(so, os.path.join(tmp, "ember", "_core"))
    sys.path.insert(0, tmp)
    import ember  # noqa

    return ember


def main():
    em = import_reference()
    T = em.Tensor
    out = {}
    for name, (B, H, Lq, Lk, D, causal, seed, bwd) in CASES.items():
        q = normal(seed, (B, H, Lq, D))
        k = normal(seed + 100, (B, H, Lk, D))
        v = normal(seed + 200, (B, H, Lk, D))
        scale = float(1.0 / np.sqrt(D))
        tq, tv = T(q), T(v)
        tkT = T(np.ascontiguousarray(np.swapaxes(k, -1, -2)))
        s = (tq @ tkT) * scale
        if causal:
            i = np.arange(Lq)[:, None]
            j = np.arange(Lk)[None, :]
            mask = np.where(j > i + (Lk - Lq), -np.inf, 0.0).astype(np.float32)
            s = s + T(mask)
        p = em.softmax(s, axis=-1)
        o = p @ tv
        mx = em.amax(s, axis=-1, keepdims=True)
        se = em.sum(em.exp(s - mx), axis=-1, keepdims=True)
        lse = mx.to_np().astype(np.float64) + np.log(se.to_np().astype(np.float64))
        out[name + "/meta"] = np.array([B, H, Lq, Lk, D, int(causal), seed], np.int64)
        out[name + "/scale"] = np.float32(scale)
        out[name + "/out"] = o.to_np()
        out[name + "/lse"] = lse[..., 0].astype(np.float32)
        if bwd:
            g = normal(seed + 300, (B, H, Lq, D))
            tg = T(g)
            pn = p.to_np()
            dv = T(np.ascontiguousarray(np.swapaxes(pn, -1, -2))) @ tg
            dp = tg @ T(np.ascontiguousarray(np.swapaxes(v, -1, -2)))
            delta = em.sum(dp * p, axis=-1, keepdims=True)
            ds = (p * (dp - delta)) * scale
            dq = ds @ T(k)
            dk = T(np.ascontiguousarray(np.swapaxes(ds.to_np(), -1, -2))) @ tq
            out[name + "/dq"], out[name + "/dk"], out[name + "/dv"] = dq.to_np(), dk.to_np(), dv.to_np()
        print(name, "ok", out[name + "/out"].shape)
    np.savez_compressed(os.path.join(HERE, "attention_golden.npz"), **out)

    # The reference's Linear layer: weights w = 0.1*N(0,1) (seed+1), bias N(0,1) (seed+2, or the
    # layer's own zeros), input N(0,1) (seed), upstream gradient N(0,1) (seed+3).
    lin = {}
    for name, (m, k, n, seed, with_bias) in LINEAR_CASES.items():
        layer = em.nn.Linear(k, n)
        layer.w = T(normal(seed + 1, (k, n)) * np.float32(0.1))
        if with_bias:
            layer.b = T(normal(seed + 2, (n,)))
        y = layer(T(normal(seed, (m, k))), True)
        gx = layer.backward(T(normal(seed + 3, (m, n))))
        gw, gb = layer.gradients()
        lin[name + "/meta"] = np.array([m, k, n, seed, int(with_bias)], np.int64)
        lin[name + "/y"], lin[name + "/gx"], lin[name + "/gw"], lin[name + "/gb"] = (
            y.to_np(), gx.to_np(), gw.to_np(), gb.to_np())
        print(name, "ok", lin[name + "/y"].shape)
    np.savez_compressed(os.path.join(HERE, "linear_golden.npz"), **lin)

    sm = {}
    for name, (rows, cols, seed) in SOFTMAX_CASES.items():
        x = normal(seed, (rows, cols)) * np.float32(3.0)
        target = np.zeros((rows, cols), np.float32)
        target[np.arange(rows), (7 * np.arange(rows)) % cols] = 1.0
        loss_fn = em.loss.CrossEntropyLoss()
        loss = loss_fn.forward(T(x), T(target))
        sm[name + "/meta"] = np.array([rows, cols, seed], np.int64)
        sm[name + "/softmax"] = em.softmax(T(x), axis=-1).to_np()
        sm[name + "/loss"] = np.float64(loss)
        sm[name + "/probs"] = loss_fn.probs.to_np()
        sm[name + "/grad"] = loss_fn.backward().to_np()
        print(name, "ok", float(loss))
    np.savez_compressed(os.path.join(HERE, "softmax_golden.npz"), **sm)


if __name__ == "__main__":
    main()
