"""CPU, two gloo ranks: the sequence-parallel hand-off protocol (`lethe_b200.parallel.sp_forward` /
`sp_backward`) driven by the oracle reproduces the single-process result, and the (batch x head)
sharding helper partitions without overlap."""

import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from lethe_b200.parallel import shard_batch_heads, sp_backward, sp_forward
from oracle.gdn_oracle import chunk_backward, chunk_forward


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _inputs(gate):
    gen = torch.Generator().manual_seed(5)
    B, L, H, K, V = 1, 128, 2, 16, 8
    dt = torch.float64
    q, k = torch.randn(B, L, H, K, generator=gen, dtype=dt), torch.randn(B, L, H, K, generator=gen, dtype=dt)
    v, do = torch.randn(B, L, H, V, generator=gen, dtype=dt), torch.randn(B, L, H, V, generator=gen, dtype=dt)
    beta = torch.rand(B, L, H, generator=gen, dtype=dt)
    g = -torch.rand(*((B, L, H, K) if gate == "channel" else (B, L, H)), generator=gen, dtype=dt)
    h0 = torch.randn(B, H, K, V, generator=gen, dtype=dt)
    dhT = torch.randn(B, H, K, V, generator=gen, dtype=dt)
    return q, k, v, g, beta, h0, do, dhT


def _worker(rank, world, port, gate):
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        q, k, v, g, beta, h0, do, dhT = _inputs(gate)
        L = q.shape[1]
        sl = slice(rank * L // world, (rank + 1) * L // world)
        loc = [t[:, sl].contiguous() for t in (q, k, v, g, beta, do)]
        like = torch.empty_like(h0)
        box = {}

        def scan(h_in):
            box["st"] = chunk_forward(loc[0], loc[1], loc[2], loc[3], loc[4], h_in, C=16)
            return box["st"].h[:, :, -1].contiguous()

        hT = sp_forward(lambda: None, scan, lambda: None, h0, like)

        def scan_b(dh_in):
            box["gr"], _ = chunk_backward(box["st"], loc[5], dh_in)
            return box["gr"].dh0.contiguous()

        dh0 = sp_backward(lambda: None, scan_b, lambda: None, dhT, like)
        # single-process answer
        st = chunk_forward(q, k, v, g, beta, h0, C=16)
        gr, _ = chunk_backward(st, do, dhT)
        assert torch.allclose(box["st"].o, st.o[:, sl], atol=1e-11)
        for n in ("dq", "dk", "dv", "dg", "dbeta"):
            assert torch.allclose(getattr(box["gr"], n), getattr(gr, n)[:, sl], atol=1e-10), n
        if rank == world - 1:
            assert torch.allclose(hT, st.h[:, :, -1], atol=1e-11)
        if rank == 0:
            assert torch.allclose(dh0, gr.dh0, atol=1e-10)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("gate", ["scalar", "channel"])
def test_sequence_parallel_protocol_two_ranks(gate):
    mp.spawn(_worker, args=(2, _free_port(), gate), nprocs=2, join=True)


def _silent_worker(rank, world, port, q):
    """Rank 0 joins the group and then never sends its boundary state (it "hangs" before its scan);
    rank 1 must get a HandoffTimeout from sp_forward, not wait for ever."""
    import datetime
    import time

    from lethe_b200.parallel import HandoffTimeout

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=60))
    try:
        like = torch.zeros(1, 2, 16, 8, dtype=torch.float64)
        if rank == 0:
            time.sleep(6.0)                      # alive, but silent for longer than its neighbour waits
            q.put(("rank0", "stayed silent"))
        else:
            t0 = time.time()
            try:
                sp_forward(lambda: None, lambda h: h, lambda: None, None, like, timeout_s=1.5)
                q.put(("rank1", "returned"))
            except HandoffTimeout as e:
                q.put(("rank1", f"timeout after {time.time() - t0:.1f}s: {str(e)[:60]}"))
    finally:
        try:
            dist.destroy_process_group()
        except Exception:     # noqa: BLE001  (the group may already be broken by the expired wait)
            pass


def test_silent_neighbour_surfaces_as_timeout_not_hang():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_silent_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=60) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
    assert got["rank0"] == "stayed silent"
    assert got["rank1"].startswith("timeout after"), got
    waited = float(got["rank1"].split()[2].rstrip("s:"))
    assert 1.0 <= waited <= 5.5, got            # gave up near its own limit, before the neighbour woke up


def test_shard_batch_heads():
    seen = set()
    for r in range(8):
        bs, hs = shard_batch_heads(16, 32, r, 8)
        for b in range(*bs.indices(16)):
            for h in range(*hs.indices(32)):
                assert (b, h) not in seen
                seen.add((b, h))
    assert len(seen) == 16 * 32
    bs, hs = shard_batch_heads(1, 32, 3, 8)
    assert (bs.start, bs.stop, hs.start, hs.stop) == (0, 1, 12, 16)
    with pytest.raises(ValueError):
        shard_batch_heads(3, 5, 0, 2)
