"""Two GPUs (skipped on a single-GPU box): sequence-parallel and (batch x head)-sharded runs of the
CUDA op are bitwise equal to the single-GPU run on the same inputs."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from lethe_b200 import ops
from lethe_b200.parallel import SequenceParallelGdn, shard_batch_heads
from lethe_b200.synth import make_inputs

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")]


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, gate):
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            device_id=dev)
    try:
        B, L, H, K, V = 2, 512, 4, 128, 64
        inp = make_inputs(B, L, H, K, V, gate=gate, delta=True, seed=31)
        d = {n: t.to(dev) for n, t in inp.items()}
        dhT = 0.1 * torch.randn(B, H, K, V, generator=torch.Generator().manual_seed(32)).to(dev)
        scale = K ** -0.5
        gate_code = ops.GATE_CHANNEL if gate == "channel" else ops.GATE_SCALAR
        # single-GPU answer, computed by every rank for itself
        full = ops.GdnBuffers(B, L, H, K, V, gate_code, True, dev)
        ops.forward_into(full, d["q"], d["k"], d["v"], d["g"], d["beta"], d["h0"], scale)
        ops.backward_into(full, d["q"], d["k"], d["v"], d["g"], d["beta"], d["h0"], d["do"], dhT, scale)
        torch.cuda.synchronize()
        # ---- sequence parallel
        Ll = L // world
        sl = slice(rank * Ll, (rank + 1) * Ll)
        loc = {n: d[n][:, sl].contiguous() for n in ("q", "k", "v", "g", "beta", "do")}
        sp = SequenceParallelGdn(B, Ll, H, K, V, gate_code, True, dev)
        o, hT = sp.forward(loc["q"], loc["k"], loc["v"], loc["g"], loc["beta"], d["h0"], scale)
        dq, dk, dv, dg, dbeta, dh0 = sp.backward(loc["do"], dhT)
        torch.cuda.synchronize()
        ops.check_status(sp.buf.status)
        assert torch.equal(o, full.o[:, sl])
        for got, ref in ((dq, full.dq), (dk, full.dk), (dv, full.dv), (dg, full.dg), (dbeta, full.dbeta)):
            assert torch.equal(got, ref[:, sl])
        if rank == world - 1:
            assert torch.equal(hT, full.hT)
        if rank == 0:
            assert torch.equal(dh0, full.dh0)
        # ---- (batch x head) sharding: no communication at all
        bs, hs = shard_batch_heads(B, H, rank, world)
        sh = {n: d[n][bs][:, :, hs].contiguous() for n in ("q", "k", "v", "g", "beta", "do")}
        h0s = d["h0"][bs][:, hs].contiguous()
        Bs, Hs = sh["q"].shape[0], sh["q"].shape[2]
        part = ops.GdnBuffers(Bs, L, Hs, K, V, gate_code, True, dev)
        ops.forward_into(part, sh["q"], sh["k"], sh["v"], sh["g"], sh["beta"], h0s, scale)
        ops.backward_into(part, sh["q"], sh["k"], sh["v"], sh["g"], sh["beta"], h0s, sh["do"],
                          dhT[bs][:, hs].contiguous(), scale)
        torch.cuda.synchronize()
        assert torch.equal(part.o, full.o[bs][:, :, hs])
        assert torch.equal(part.dk, full.dk[bs][:, :, hs])
        assert torch.equal(part.dg, full.dg[bs][:, :, hs])
        assert torch.equal(part.dh0, full.dh0[bs][:, hs])
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("gate", ["scalar", "channel"])
def test_two_gpu_modes_match_single_gpu(gate):
    mp.spawn(_worker, args=(2, _free_port(), gate), nprocs=2, join=True)
