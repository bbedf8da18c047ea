"""The multi-GPU orchestration (row-block split, broadcast of B, all-gather of B's norm map, gather of the C slabs)
run as two gloo ranks on CPU.  The per-rank plan is a stand-in backed by the CPU checker; the class under test
(`ShardedSpamm`) is the one the GPU path uses."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import signed_decay


class CpuPlan:
    """Same surface as SpammPlan for what ShardedSpamm touches, CPU tensors instead of device buffers."""

    def __init__(self, M, K, N, begin, count):
        from cuspamm_b200 import BUF_A, BUF_B, BUF_C, BUF_COUNTS, BUF_NORM_A, BUF_NORM_B

        self.M, self.K, self.N = M, K, N
        self.row_tile_begin, self.row_tile_count = begin, count
        self.rows = count * 32
        self.t = {BUF_A: torch.zeros(self.rows, K), BUF_B: torch.zeros(K, N), BUF_C: torch.zeros(self.rows, N),
                  BUF_NORM_A: torch.zeros(count, K // 32), BUF_NORM_B: torch.full((K // 32, N // 32), -1.0),
                  BUF_COUNTS: torch.zeros(count, N // 32, dtype=torch.int32)}
        self.ids = (BUF_A, BUF_B, BUF_C, BUF_NORM_A, BUF_NORM_B, BUF_COUNTS)

    def as_tensor(self, which):
        return self.t[which]

    def upload(self, a_rows=None, b=None):
        A, B = self.ids[0], self.ids[1]
        if a_rows is not None:
            self.t[A].copy_(torch.from_numpy(a_rows))
        if b is not None:
            self.t[B].copy_(torch.from_numpy(b))

    def norms_share(self, b_begin, b_count):
        from oracle import oracle as O

        A, B, _, NA, NB, _ = self.ids
        self.t[NA].copy_(torch.from_numpy(O.norm_map(self.t[A].numpy())))
        if b_count:
            share = O.norm_map(self.t[B].numpy()[b_begin * 32:(b_begin + b_count) * 32])
            self.t[NB][b_begin:b_begin + b_count].copy_(torch.from_numpy(share))

    def norms(self):
        self.norms_share(0, self.K // 32)

    def build_lists(self, tau):
        from oracle import oracle as O

        _, _, _, NA, NB, CNT = self.ids
        counts, self.offsets, self.kidx = O.lists(self.t[NA].numpy(), self.t[NB].numpy(), tau)
        self.t[CNT].copy_(torch.from_numpy(counts))

    def pack(self):
        from oracle import oracle as O

        self.Ah = O.round_to_half(self.t[self.ids[0]].numpy())
        self.Bh = O.round_to_half(self.t[self.ids[1]].numpy())

    def gated_multiply(self):
        from oracle import oracle as O

        self.t[self.ids[2]].copy_(torch.from_numpy(O.gated_multiply(self.Ah, self.Bh, self.offsets, self.kidx)))

    def counts(self):
        c = self.t[self.ids[5]].numpy()
        return c, int(c.sum())

    def sync(self):
        pass


def _worker(rank, world, port, n, tau, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from cuspamm_b200 import ShardedSpamm

        A = signed_decay(n, 0.04, 31)
        B = signed_decay(n, 0.05, 32)
        sh = ShardedSpamm(n, n, n, plan_factory=CpuPlan)
        b, c = sh.row_tile_begin, sh.row_tile_count
        # only rank 0 holds B on the host; the others must receive it by broadcast
        sh.distribute(np.ascontiguousarray(A[b * 32:(b + c) * 32]), B if rank == 0 else None)
        sh.run(tau)
        S = sh.survivors()
        full = sh.gather_c(0)
        if rank == 0:
            np.save(os.path.join(out_dir, "C.npy"), full.numpy())
            np.save(os.path.join(out_dir, "S.npy"), np.array([S]))
        else:
            assert full is None
            assert (sh.plan.as_tensor(4) >= 0).all()      # every share of B's norm map arrived
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,n", [(2, 256), (2, 96)])
def test_two_ranks_reproduce_the_single_rank_result(tmp_path, oracle, world, n):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    tau = 0.3
    mp.spawn(_worker, args=(world, port, n, tau, str(tmp_path)), nprocs=world, join=True)
    A = signed_decay(n, 0.04, 31)
    B = signed_decay(n, 0.05, 32)
    C_ref, S_ref = oracle.spamm(A, B, tau)
    assert int(np.load(tmp_path / "S.npy")[0]) == S_ref
    assert np.array_equal(np.load(tmp_path / "C.npy"), C_ref)


def test_balanced_row_blocks_properties():
    """The survivor-balanced split: contiguous, complete, on macro-tile boundaries, never worse than the even split."""
    from cuspamm_b200 import balanced_row_blocks, row_blocks

    rng = np.random.default_rng(5)
    for T, world in [(1024, 8), (1024, 4), (512, 2), (100, 3), (64, 8), (7, 4), (3, 8), (0, 2)]:
        w = rng.random(T) ** 4 * 1000 + 5
        blocks = balanced_row_blocks(w, world)
        assert len(blocks) == world and blocks[0][0] == 0 and sum(c for _, c in blocks) == T
        assert all(blocks[i][0] + blocks[i][1] == blocks[i + 1][0] for i in range(world - 1))
        if T >= 4 * world:
            assert all(b % 4 == 0 for b, _ in blocks)
            assert all(c > 0 for _, c in blocks)
        load = lambda bl: max((w[b:b + c].sum() for b, c in bl), default=0.0)   # noqa: E731
        assert load(blocks) <= load(row_blocks(T, world)) + 1e-9
    # a ramp: the even split is 1.75x the mean at 8 blocks, the balanced one within a few percent
    w = np.arange(1024.0) + 1
    blocks = balanced_row_blocks(w, 8)
    assert max(w[b:b + c].sum() for b, c in blocks) <= 1.05 * w.sum() / 8
    assert balanced_row_blocks(np.zeros(64), 4) == row_blocks(64, 4)


def _worker_balanced(rank, world, port, n, tau, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from cuspamm_b200 import ShardedSpamm, balanced_row_blocks

        A = signed_decay(n, 0.04, 31)
        A[: n // 4] *= np.float32(50.0)          # the first quarter of the rows keeps far more products
        B = signed_decay(n, 0.05, 32)

        def run(blocks):
            sh = ShardedSpamm(n, n, n, plan_factory=CpuPlan, blocks=blocks)
            b, c = sh.row_tile_begin, sh.row_tile_count
            sh.distribute(np.ascontiguousarray(A[b * 32:(b + c) * 32]), B if rank == 0 else None)
            sh.run(tau)
            return sh

        sh = run(None)
        per_row = sh.row_survivors()
        assert per_row.shape == (n // 32,) and int(per_row.sum()) == sh.survivors()
        blocks = balanced_row_blocks(per_row + 1.0, world)
        assert blocks != sh.blocks and blocks[0][1] < sh.blocks[0][1]      # the heavy rows get the smaller block
        sh2 = run(blocks)
        assert sh2.survivors() == sh.survivors()
        full = sh2.gather_c(0)
        if rank == 0:
            np.save(os.path.join(out_dir, "C.npy"), full.numpy())
            np.save(os.path.join(out_dir, "blocks.npy"), np.array(blocks))
    finally:
        dist.destroy_process_group()


def test_survivor_balanced_partition_gives_the_same_product(tmp_path, oracle):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    n, tau, world = 512, 50.0, 2
    mp.spawn(_worker_balanced, args=(world, port, n, tau, str(tmp_path)), nprocs=world, join=True)
    A = signed_decay(n, 0.04, 31)
    A[: n // 4] *= np.float32(50.0)
    B = signed_decay(n, 0.05, 32)
    C_ref, _ = oracle.spamm(A, B, tau)
    assert np.array_equal(np.load(tmp_path / "C.npy"), C_ref)
    blocks = np.load(tmp_path / "blocks.npy")
    assert blocks[0][1] != blocks[1][1]


def test_balanced_row_blocks_random_weights():
    """Property check over random weight vectors: a complete contiguous split that is never worse than the even one,
    and within one unit's weight of the ideal share."""
    from hypothesis import given, settings, strategies as st

    from cuspamm_b200 import balanced_row_blocks, row_blocks

    @settings(max_examples=200, deadline=None, derandomize=True)
    @given(st.lists(st.floats(min_value=0.0, max_value=1e6, allow_nan=False), min_size=1, max_size=300),
           st.integers(min_value=1, max_value=8))
    def check(weights, world):
        w = np.asarray(weights, dtype=np.float64)
        T = len(w)
        blocks = balanced_row_blocks(w, world)
        assert len(blocks) == world and blocks[0][0] == 0 and sum(c for _, c in blocks) == T
        assert all(c >= 0 for _, c in blocks)
        assert all(blocks[i][0] + blocks[i][1] == blocks[i + 1][0] for i in range(world - 1))
        load = lambda bl: max((w[b:b + c].sum() for b, c in bl), default=0.0)   # noqa: E731
        assert load(blocks) <= load(row_blocks(T, world)) * (1 + 1e-9) + 1e-9
        unit = 4 if T >= 4 * world else 1
        heaviest_unit = max(w[u:u + unit].sum() for u in range(0, T, unit))
        assert load(blocks) <= w.sum() / world + heaviest_unit + 1e-6 * max(1.0, w.sum())

    check()
