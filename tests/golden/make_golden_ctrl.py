"""Golden fixtures for the controller-conditioning path, from the reference's own CPU oracles.

    python tests/golden/make_golden_ctrl.py /path/to/reference

Writes ``ctrl.npz`` beside this file (the other fixtures come from ``make_golden.py`` and are not touched):
plain RMSNorm and elementwise add through their numpy references, and ``MLPFusion`` /
``ControllerInputEmbedding`` composed from the GEMM and SiLU references in the order the reference's
modules launch them (``src/quark/nn/layers.py:760-822``).  ``tests/test_oracle_golden.py`` replays the
file against ``oracle/``.
"""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent


def _bf16(a):
    return (np.ascontiguousarray(a, dtype=np.float32).view(np.uint32) >> 16).astype(np.uint16)


def main(ref_root: str) -> None:
    sys.path.insert(0, str(Path(ref_root) / "src"))
    from quark.kernels.elementwise.reference import elementwise_reference_numpy
    from quark.kernels.elementwise.spec import ElementwiseSpec
    from quark.kernels.gemm.reference import gemm_reference_numpy
    from quark.kernels.gemm.spec import GemmSpec
    from quark.kernels.rmsnorm.reference import rmsnorm_reference_numpy
    from quark.kernels.rmsnorm.spec import RMSNormSpec
    from quark.kernels.silu.reference import silu_reference_numpy
    from quark.kernels.silu.spec import SiLUSpec

    rng = np.random.default_rng(0xC7A1)
    M, D = 32, 256
    X = _bf16(rng.standard_normal((M, D)))
    Y = _bf16(rng.standard_normal((M, D)))
    cond = _bf16(rng.standard_normal((1, D)))
    out = dict(X=X, Y=Y, cond=cond)
    out["rmsnorm"] = rmsnorm_reference_numpy(RMSNormSpec(B=M, D=D, dtype="bf16", eps=1e-6), X=X)
    out["rmsnorm_row"] = rmsnorm_reference_numpy(RMSNormSpec(B=1, D=D, dtype="bf16", eps=1e-6), X=cond)
    out["add"] = elementwise_reference_numpy(ElementwiseSpec(N=M * D, dtype="bf16", op="add"), X=X.reshape(-1), Y=Y.reshape(-1)).reshape(M, D)

    # MLPFusion: h_c = fc1_c(cond); h = silu(fc1_x(x) + h_c); y = fc2(h)
    Wx, Wc, W2 = (_bf16(0.08 * rng.standard_normal((D, D))) for _ in range(3))
    out.update(Wx=Wx, Wc=Wc, W2=W2)
    h_c = gemm_reference_numpy(GemmSpec(M=1, N=D, K=D), A=cond, B=Wc)
    h = gemm_reference_numpy(GemmSpec(M=M, N=D, K=D, has_bias=True), A=X, B=Wx, Bias=np.asarray(h_c).reshape(-1))
    h = silu_reference_numpy(SiLUSpec(N=M * D), X=np.asarray(h).reshape(-1)).reshape(M, D)
    out["mlp_fusion"] = gemm_reference_numpy(GemmSpec(M=M, N=D, K=D), A=h, B=W2)

    # ControllerInputEmbedding with 29 buttons -> 32 padded inputs, hidden 4 * 64
    d, n_buttons = 64, 29
    padded = (n_buttons + 3 + 15) // 16 * 16
    row = np.zeros((1, padded), np.float32)
    row[0, 0], row[0, 1] = 0.25, -0.5
    row[0, 2 + 3] = row[0, 2 + 17] = 1.0
    row[0, 2 + n_buttons] = -1.0
    ctrl = _bf16(row)
    W1 = _bf16(0.2 * rng.standard_normal((4 * d, padded)))
    W2e = _bf16(0.1 * rng.standard_normal((d, 4 * d)))
    e = gemm_reference_numpy(GemmSpec(M=1, N=4 * d, K=padded), A=ctrl, B=W1)
    e = silu_reference_numpy(SiLUSpec(N=4 * d), X=np.asarray(e).reshape(-1)).reshape(1, 4 * d)
    out.update(ctrl_input=ctrl, We1=W1, We2=W2e)
    out["ctrl_emb"] = gemm_reference_numpy(GemmSpec(M=1, N=d, K=4 * d), A=e, B=W2e)
    np.savez_compressed(HERE / "ctrl.npz", **{k: np.asarray(v) for k, v in out.items()})
    print("wrote ctrl.npz:", sorted(out))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden_ctrl.py <checkout of the reference project>")
    main(sys.argv[1])
