"""GPU: the reference project's 12-gate Kernel Contract battery, run UNCHANGED (``run_all_gates``,
``verifier/contracts.py:747-790`` of the reference, imported from ``oracle/_ref``) on this library's
backward entry point ``lethe_b200.ops.gdn2_backward`` through the reference's own single-gradient
adapters (``verifier/op_harness.py:714-760``), at the head size the kernels are built for
(d_k = d_v = 128; the reference runs its battery at head size 4 on its eager CPU path).

Only gate ARGUMENTS are overridden, as the reference's harness does for its own ops
(``GDN2_BWD_GATE_OVERRIDES``): shapes whose model width is a multiple of 128, and the north-star
tolerance (5e-3 of the reference's largest magnitude) where a gate takes one.

What each gate must do here is stated below, gate by gate.  Seven gates pass.  Five cannot pass for ANY
kernel of this design, and the test pins that they fail for exactly that reason rather than for another:
  CMP-02  differentiates the candidate a second time in fp64: the backward is first-order only and there
          is no eager fallback to route a second derivative to (the reference falls back to its oracle);
  PRC-01  demands 1e-5 agreement for fp32 inputs: operands enter the tensor cores as 16-bit values;
  EXC-01  demands NaN / Inf masks equal to a token-serial evaluation: a chunkwise kernel multiplies masked
          (zero) coefficients with every row of the 64-token chunk, so a NaN reaches the whole chunk;
  EXC-02  demands the reference's exact pattern of zeros for upstream gradients of 1e-40: which products
          underflow to zero depends on the order of fp32 operations of the eager token loop;
  RES-01  calls the candidate on CPU tensors: there is no CPU path by design.
"""

import pytest
import torch

from lethe_b200 import ops

from .refimport import reference
from .wsview import report

pytestmark = pytest.mark.gpu

HEAD = 128
TOL = 5e-3
SHAPE = (2, 64, 2 * HEAD)             # [batch, tokens, heads * 128]: the reference oracle is a token loop

OVERRIDES = {
    "gate_cmp_01_input_variation": {"shape": SHAPE, "atol": TOL, "rtol": 0.0, "n_random": 4},
    "gate_cmp_02_gradient_correctness": {"shape": (1, 64, HEAD)},
    "gate_cmp_03_shape_polymorphism": {"atol": TOL, "rtol": 0.0,
                                       "shapes": [(1, 64, HEAD), (2, 128, 2 * HEAD), (1, 192, HEAD), (3, 64, 2 * HEAD)]},
    # the kernel's native input type: the gate scales its tolerance to that type's rounding
    "gate_ord_01_reduction_order_tolerance": {"shape": (2, 256, 2 * HEAD), "dtype": torch.bfloat16,
                                              "reduction_elements": 512},
    "gate_ord_02_atomic_determinism": {"shape": SHAPE},
    "gate_ord_03_noncommutative_reduction": {"shape": (1, 512, HEAD), "atol": 3e-3, "rtol": 3e-3},
    "gate_prc_01_precision_regime": {"shape": SHAPE},
    "gate_prc_02_mixed_precision_accumulation": {"shape": (1, 512, 2 * HEAD), "atol": TOL, "rtol": 0.0,
                                                 "scale_atol_by_ref_inf": True},
    "gate_exc_01_exceptional_values": {"shape": SHAPE},
    "gate_exc_02_subnormal_handling": {"shape": SHAPE},
    "gate_res_01_memory_residency": {"shape": SHAPE},
    # per-thread registers, dynamic shared memory and tensor-memory columns of the largest kernels
    # (nvcc -Xptxas -v of csrc/: see profiles/)
    "gate_res_02_resource_limits": {"resource_meta": {"n_regs": 128, "shared_bytes": 214 * 1024, "tmem_elems": 512}},
}

MUST_PASS = ("gate_cmp_01_input_variation", "gate_cmp_03_shape_polymorphism",
             "gate_ord_01_reduction_order_tolerance", "gate_ord_02_atomic_determinism",
             "gate_ord_03_noncommutative_reduction", "gate_prc_02_mixed_precision_accumulation",
             "gate_res_02_resource_limits")
FAILS_BY_DESIGN = {
    "gate_cmp_02_gradient_correctness": "gradcheck",
    "gate_prc_01_precision_regime": "torch.float32",
    "gate_exc_01_exceptional_values": "mask mismatch",
    "gate_exc_02_subnormal_handling": "flush-to-zero",
    "gate_res_01_memory_residency": "device=cpu",
}


def _run(view):
    reference()
    from lethe.verifier.contracts import run_all_gates
    from lethe.verifier.op_harness import gdn2_bwd_candidate_adapter, gdn2_bwd_reference_adapter

    cand = gdn2_bwd_candidate_adapter(ops.gdn2_backward, view, headdim=HEAD)
    ref = gdn2_bwd_reference_adapter(view, headdim=HEAD)
    res = run_all_gates(cand, ref, device="cuda", gate_overrides=OVERRIDES)
    assert len(res) == 12
    for name, r in res.items():
        print(f"[{view}] {name}: {'PASS' if r.passed else 'FAIL'} - {r.reason} {r.details if not r.passed else ''}")
    report(f"contract gates {view}", {n.split('_', 2)[1] + n.split('_', 3)[2]: float(r.passed) for n, r in res.items()})
    return res


def _check(view, res):
    for name in MUST_PASS:
        assert res[name].passed, (view, name, res[name].reason, res[name].details)
    for name, why in FAILS_BY_DESIGN.items():
        r = res[name]
        text = r.reason + " " + str(r.details)
        assert not r.passed and why in text, (view, name, text)


def test_contract_gates_fast_view():
    """The view the reference's own fast check uses (grad_v, ``tests/test_op_harness_gdn2.py:114-123``)."""
    _check("grad_v", _run("grad_v"))


@pytest.mark.slow
@pytest.mark.parametrize("view", ["grad_q", "grad_k", "grad_g", "grad_b", "grad_w"])
def test_contract_gates_all_views(view):
    _check(view, _run(view))
