"""Worker of tests/test_gpu_sharded.py: one rank per GPU under torchrun; rank 0 checks the gathered C."""
import os
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))


def main():
    import torch
    import torch.distributed as dist

    from conftest import rel_fro
    from cuspamm_b200 import ShardedSpamm, gen_uniform_alg

    n, tau = int(sys.argv[1]), float(sys.argv[2])
    exchange = sys.argv[3] if len(sys.argv) > 3 else "nccl"
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank = dist.get_rank()
    sh = ShardedSpamm(n, n, n, exchange=exchange)
    b0, cnt = sh.row_tile_begin, sh.row_tile_count
    A_rows = gen_uniform_alg(3, cnt * 32, n, row_begin=b0 * 32)     # algebraic decay with random magnitudes
    B = gen_uniform_alg(4, n, n) if rank == 0 else None
    for _ in range(3):                                              # several steps: buffers and flags are reused
        sh.distribute(A_rows, B)
        sh.run(tau)
        S = sh.survivors()
        full = sh.gather_c(0)
    # host matrices in and out on every rank: its rows of A, its rows of B, its rows of C back (twice: buffers reused)
    r0, rows = sh.b_rows()
    B_mine = gen_uniform_alg(4, rows, n, row_begin=r0)
    for _ in range(2):
        C_mine, st = sh.multiply(A_rows, B_mine, tau)
    parts = [None] * dist.get_world_size()
    dist.all_gather_object(parts, (C_mine, st["survivors"]))
    ok = True
    if rank == 0:
        from oracle import oracle as O

        A = gen_uniform_alg(3, n, n)
        C_ref, S_ref = O.spamm(A, B, tau)
        err = rel_fro(full.cpu().numpy(), C_ref)
        err_h = rel_fro(np.vstack([p[0] for p in parts]), C_ref)
        S_h = sum(p[1] for p in parts)
        ok = (S == S_ref) and err <= 1e-3 and (S_h == S_ref) and err_h <= 1e-3
        print(f"exchange={exchange} push={sh._push} sharded world={dist.get_world_size()} n={n} S={S} S_ref={S_ref} "
              f"rel_fro={err:.3e} host_to_host: S={S_h} rel_fro={err_h:.3e} ok={ok}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
