"""The L2 normalisation of q and k and its vector-Jacobian product as CUDA kernels, against PyTorch in
fp64 (same formula as the reference, ``gdn_backward.py:9-10``: epsilon inside the root), and through
the differentiable op with ``use_qk_l2norm=True`` against the token-serial fp64 oracle."""
import pytest
import torch

from lethe_b200 import ops
from lethe_b200.synth import make_inputs
from oracle.gdn_oracle import scale_rel, serial_forward

from .wsview import report

pytestmark = pytest.mark.gpu


def _ref(x, eps=1e-6):
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + eps)


@pytest.mark.parametrize("norm_dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("D,rows", [(128, (3, 37, 5)), (64, (2, 129, 3)), (128, (1, 1, 1))])
def test_forward_and_vjp_against_fp64(dtype, D, rows, norm_dtype):
    """Normalised rows and their gradients as fp16 (the default: the operand type of the GDN kernels,
    one rounding) and as bf16."""
    gen = torch.Generator().manual_seed(5)
    q = (torch.randn(*rows, D, generator=gen) * 3).to(dtype)
    k = torch.randn(*rows, D, generator=gen).to(dtype)
    k[0, 0] = 0                                             # a zero row: epsilon decides the result
    dqn = torch.randn(*rows, D, generator=gen).to(norm_dtype)
    dkn = torch.randn(*rows, D, generator=gen).to(norm_dtype)

    q64 = q.double().requires_grad_(True)
    k64 = k.double().requires_grad_(True)
    qn_ref, kn_ref = _ref(q64), _ref(k64)
    dq_ref, dk_ref = torch.autograd.grad((qn_ref, kn_ref), (q64, k64), (dqn.double(), dkn.double()))

    dev = torch.device("cuda")
    qd, kd = q.to(dev), k.to(dev)
    qn, kn = ops.l2norm_qk_raw(qd, kd, norm_dtype=norm_dtype)
    assert qn.dtype == norm_dtype and kn.dtype == norm_dtype
    dq, dk = ops.l2norm_qk_vjp_raw(qd, kd, dqn.to(dev), dkn.to(dev))
    dq, dk = dq.to(dtype), dk.to(dtype)
    if norm_dtype == torch.float16:                          # the differentiable wrapper: fp16 rows
        qr, kr = qd.clone().requires_grad_(True), kd.clone().requires_grad_(True)
        qn2, kn2 = ops.l2norm_qk(qr, kr)
        assert qn2.dtype == torch.float16 and torch.equal(qn2, qn) and torch.equal(kn2, kn)
        dq2, dk2 = torch.autograd.grad((qn2, kn2), (qr, kr), (dqn.to(dev), dkn.to(dev)))
        assert dq2.dtype == dtype and torch.equal(dq2, dq) and torch.equal(dk2, dk)
    errs = {"qn": scale_rel(qn.double().cpu(), qn_ref.detach()), "kn": scale_rel(kn.double().cpu(), kn_ref.detach()),
            "dq": scale_rel(dq.double().cpu(), dq_ref), "dk": scale_rel(dk.double().cpu(), dk_ref)}
    report(f"l2norm {dtype} D={D} rows={rows}", errs)
    out_tol = 2.0 ** -8 if norm_dtype == torch.bfloat16 else 2.0 ** -11      # rounding of the outputs
    assert errs["qn"] <= out_tol and errs["kn"] <= out_tol
    grad_tol = 2.0 ** -8 if dtype == torch.bfloat16 else 1e-5
    assert errs["dq"] <= grad_tol and errs["dk"] <= grad_tol


@pytest.mark.parametrize("gate,delta", [("scalar", True), ("channel", True), ("scalar", False)])
def test_op_with_l2norm_against_serial_oracle(gate, delta):
    B, L, H, K, V = 1, 192, 2, 128, 64
    inp = make_inputs(B, L, H, K, V, gate=gate, delta=delta, seed=21)
    gen = torch.Generator().manual_seed(22)
    inp["q"] = (torch.randn(B, L, H, K, generator=gen) * 2).to(torch.bfloat16)     # not pre-normalised
    inp["k"] = (torch.randn(B, L, H, K, generator=gen) * 0.5).to(torch.bfloat16)
    f64 = {n: (None if t is None else t.double()) for n, t in inp.items()}
    # oracle with the normalisation inside the differentiated function
    q64 = f64["q"].clone().requires_grad_(True)
    k64 = f64["k"].clone().requires_grad_(True)
    v64 = f64["v"].clone().requires_grad_(True)
    o_ref, _ = serial_forward(_ref(q64), _ref(k64), v64, f64["g"], f64["beta"], f64["h0"])
    dq_ref, dk_ref, dv_ref = torch.autograd.grad(o_ref, (q64, k64, v64), f64["do"])

    dev = torch.device("cuda")
    d = {n: (None if t is None else t.to(dev)) for n, t in inp.items()}
    qd, kd, vd = (d[n].clone().requires_grad_(True) for n in ("q", "k", "v"))
    o, _ = ops.gdn_chunk(qd, kd, vd, d["g"], d["beta"], d["h0"], use_qk_l2norm=True)
    dq, dk, dv = torch.autograd.grad(o, (qd, kd, vd), d["do"])
    errs = {"o": scale_rel(o.double().cpu(), o_ref.detach()), "dq": scale_rel(dq.double().cpu(), dq_ref),
            "dk": scale_rel(dk.double().cpu(), dk_ref), "dv": scale_rel(dv.double().cpu(), dv_ref)}
    report(f"op l2norm gate={gate} delta={delta}", errs)
    # the normalised rows are formed in fp32 and rounded once, to the fp16 operand type; dq, dk come back
    # from the kernels as fp16 and meet bf16 only in the final cast to the input dtype
    assert max(errs.values()) <= 5e-3, errs
