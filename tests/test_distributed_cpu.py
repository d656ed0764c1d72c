"""world_size-2 gloo test of the column-parallel exchange on CPU: every rank
computes its shard with the oracle, the all-gather assembles the full output."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import w4a4_oracle as O
from zip_kernel_b200 import sharding, synth


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, N, K, T, token_major, out_q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        W = synth.make_container(N, K, 0.3, seed=11)
        X = synth.make_activations(T, K, seed=12)
        xs4, sx, sumx = O.quantize_activation_s4(X.numpy(), W.perm.numpy())
        S = sharding.shard_container(W, rank, world)
        sharding.check_shard_metadata(N, K, S, rank, world)
        y = O.fused_kernel_order(S.W_low_packed.numpy(), S.W_high_blocks_packed.numpy(), S.hp_row_offsets.numpy(),
                                 S.hp_col_indices.numpy(), xs4, S.scale_u4.numpy(), S.zero_u4.numpy(), sumx, sx,
                                 S.d_out, K)                               # (d_out_r, T)
        y_local = torch.from_numpy(y.T.copy() if token_major else y)
        full = sharding.gather_output(y_local, N, token_major=token_major)
        ref = O.fused_kernel_order(W.W_low_packed.numpy(), W.W_high_blocks_packed.numpy(), W.hp_row_offsets.numpy(),
                                   W.hp_col_indices.numpy(), xs4, W.scale_u4.numpy(), W.zero_u4.numpy(), sumx, sx, N, K)
        want = ref.T if token_major else ref
        out_q.put((rank, bool(np.array_equal(full.numpy().view(np.uint16), np.ascontiguousarray(want).view(np.uint16)))))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("N,token_major", [(512, True), (512, False), (640, True), (384, False)])
def test_column_parallel_gather_gloo(N, token_major):
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, N, 256, 3, token_major, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(results) == [(0, True), (1, True)]
