"""Column-parallel sharding on real GPUs: every rank runs its shard of a linear,
the fp16 shards are all-gathered - over NCCL, and through the library's own
exchange over peer memory (one kernel that stores the shard into every rank's
buffer and waits for the other ranks' flags) - and must equal the single-GPU
result bit for bit (rows of the linear are independent, so sharding changes
nothing in the arithmetic).  Needs at least two GPUs; skipped otherwise."""

import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, T, K, N, out_q):
    import torch.distributed as dist
    from zip_kernel_b200 import sharding, synth, v9_linear
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        W = synth.make_container(N, K, 0.1, seed=7, perm_seed=1)
        X = synth.make_activations(T, K, seed=8).to(dev)
        shard = sharding.shard_container(W, rank, world)
        sharding.check_shard_metadata(N, K, shard, rank, world)
        full = sharding.column_parallel_forward(X, shard.to(dev), N)
        single = v9_linear.v9_linear_forward(X, W.to(dev))
        ok = bool(torch.equal(full, single))
        # the same through the peer-memory exchange: several steps in a row (the two buffer sets alternate), both
        # output layouts, and once replayed from a CUDA graph
        pg = sharding.PeerGather(2 * T * N, device=dev)
        sd = shard.to(dev)
        for step in range(5):
            Xs = (X.float() * (1.0 + 0.25 * step)).half()
            got = sharding.column_parallel_forward(Xs, sd, N, exchange=pg)
            ok = ok and bool(torch.equal(got, v9_linear.v9_linear_forward(Xs, W.to(dev))))
        from zip_kernel_b200 import ops
        y_nt = ops.fused_dense_sparse_e2e_cuda(X, sd.perm, sd.W_low_packed, sd.W_high_blocks_packed, sd.hp_row_offsets,
                                               sd.hp_col_indices, sd.scale_u4, sd.zero_u4, sd.d_out, sd.d_in)     # (d_out_r, T)
        ok = ok and bool(torch.equal(pg.gather(y_nt, N, token_major=False), single.t()))
        from zip_kernel_b200 import _lib
        holder = _lib.WorkspaceHolder()
        side = torch.cuda.Stream()
        xg = X.clone()
        with _lib.use_workspace(holder), torch.cuda.stream(side):
            for _ in range(2):
                sharding.column_parallel_forward(xg, sd, N, exchange=pg)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                out1 = sharding.column_parallel_forward(xg, sd, N, exchange=pg).clone()
                out2 = sharding.column_parallel_forward(xg, sd, N, exchange=pg).clone()
        torch.cuda.synchronize()
        for rep in range(3):
            xg.copy_((X.float() * (2.0 + rep)).half())
            g.replay()
            torch.cuda.synchronize()
            want = v9_linear.v9_linear_forward(xg, W.to(dev))
            ok = ok and bool(torch.equal(out1, want)) and bool(torch.equal(out2, want))
        ok = ok and _lib.device_error(dev) == 0
        pg.close()
        out_q.put((rank, ok, tuple(full.shape)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("T,K,N", [(3, 512, 1024), (16, 1024, 1152)])   # equal shards; ragged shards (9 block-rows)
def test_sharded_forward_matches_single_gpu(T, K, N):
    world = 2
    if torch.cuda.device_count() < world:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, T, K, N, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=240)
    alive = [p for p in procs if p.is_alive()]
    for p in alive:
        p.kill()                      # exact processes started above
    assert not alive, "a rank did not finish"
    got = sorted(q.get(timeout=10) for _ in range(world))
    assert [g[1] for g in got] == [True] * world, got
    assert all(g[2] == (T, N) for g in got)
