"""Golden fixture for the mixture-of-experts MLP, from the reference's own CPU oracles.

    python tests/golden/make_golden_moe.py /path/to/reference

Writes ``moe.npz`` beside this file: seeded inputs, and the outputs of the reference's four numpy references
chained the way ``nn.MoE.forward`` launches them with ``routing="correct"`` (``src/quark/nn/moe.py:252-363``):
router GEMM -> ``moe_router_correct`` -> ``moe_inproj`` -> ``moe_outproj`` (f32 partials) -> ``moe_reduce``.
The slot tables of the router are also stored in the dense form this repository's oracle uses (``[E, M]`` weights,
zero where a token does not use an expert).  ``tests/test_oracle_golden.py`` replays the file against ``oracle/``.
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
    from quark.kernels.gemm.reference import gemm_reference_numpy
    from quark.kernels.gemm.spec import GemmSpec
    from quark.kernels.moe_inproj.reference import moe_inproj_reference_numpy
    from quark.kernels.moe_inproj.spec import MoeInprojSpec
    from quark.kernels.moe_outproj.reference import moe_outproj_reference_numpy
    from quark.kernels.moe_outproj.spec import MoeOutprojSpec
    from quark.kernels.moe_reduce.reference import moe_reduce_reference_numpy
    from quark.kernels.moe_reduce.spec import MoeReduceSpec
    from quark.kernels.moe_router_correct.reference import moe_router_correct_reference_numpy
    from quark.kernels.moe_router_correct.spec import MoeRouterCorrectSpec

    rng = np.random.default_rng(0x30E5)
    M, D, H, E, K = 96, 64, 96, 8, 2
    # capacity as nn.MoE computes it for routing="correct" (moe.py:120-123)
    worst = M * K + E * 31
    capacity = ((worst + E - 1) // E + 31) // 32 * 32
    X = _bf16(rng.standard_normal((M, D)))
    Wr = _bf16(0.5 * rng.standard_normal((E, D)))
    W_in = _bf16(0.1 * rng.standard_normal((E * H, D)))
    W_out = _bf16(0.1 * rng.standard_normal((E * D, H)))

    logits = gemm_reference_numpy(GemmSpec(M=M, N=E, K=D), A=X, B=Wr)  # bf16, as the router Linear stores it
    logits_f32 = (np.asarray(logits, np.uint16).astype(np.uint32) << 16).view(np.float32)
    r = moe_router_correct_reference_numpy(MoeRouterCorrectSpec(M=M, E=E, top_k=K, capacity=capacity), logits=logits_f32)
    h = moe_inproj_reference_numpy(MoeInprojSpec(M=M, D=D, H=H, n_experts=E, top_k=K, capacity=capacity), X=X, W_in=W_in,
                                   token_ids=r["token_ids"], work_list=np.where(r["work_list"] < 0, 0, r["work_list"]))  # fmt: skip
    part = moe_outproj_reference_numpy(MoeOutprojSpec(M=M, D=D, H=H, n_experts=E, top_k=K, capacity=capacity, out_dtype="f32"),
                                       h_in=h, W_out=W_out, work_list=r["work_list"])  # fmt: skip
    out = moe_reduce_reference_numpy(MoeReduceSpec(M=M, D=D, n_experts=E, capacity=capacity, top_k=K, partials_dtype="f32"),
                                     partials=part, slot_weights=r["slot_weights"], token_slot_table=r["token_slot_table"])  # fmt: skip

    # the router's slot tables in dense form: which expert owns a slot follows from the per-expert offsets
    dense = np.zeros((E, M), np.float32)
    offs = np.asarray(r["offsets"], np.int64)
    for m in range(M):
        for k in range(K):
            slot = int(r["token_slot_table"][m, k])
            e = int(np.searchsorted(offs[1:], slot, side="right"))
            assert int(r["token_ids"][slot]) == m
            dense[e, m] = r["slot_weights"][slot]
    np.savez_compressed(HERE / "moe.npz", X=X, Wr=Wr, W_in=W_in, W_out=W_out, logits=np.asarray(logits, np.uint16),
                        weights=dense, counts=np.asarray(r["counts"], np.int32), out=np.asarray(out, np.uint16),
                        geometry=np.array([M, D, H, E, K], np.int32),
                        # the router's slot tables as the reference lays them out (row tile 32)
                        slot_token_ids=np.asarray(r["token_ids"], np.int32), slot_weights=np.asarray(r["slot_weights"], np.float32),
                        slot_offsets=np.asarray(r["offsets"], np.int32), token_slot_table=np.asarray(r["token_slot_table"], np.int32),
                        work_list=np.asarray(r["work_list"], np.int32), capacity=np.array([capacity], np.int32))  # fmt: skip
    print("moe.npz:", {k: int(v) for k, v in zip("MDHEK", (M, D, H, E, K))}, "counts", r["counts"].tolist())


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    main(sys.argv[1])
