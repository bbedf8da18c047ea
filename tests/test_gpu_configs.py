"""The benchmark configurations on the GPU: exact comparison with the CPU checker where it
finishes in seconds, and size-independent properties at the full sizes (survivor counts against the checker's
count on the same norm maps, dense limit against a float matrix product of the half-rounded inputs, row blocks
that tile the result, a second call that reproduces the first bit for bit)."""
import numpy as np
import pytest

from conftest import rel_fro

pytestmark = pytest.mark.gpu
C_TOL = 1e-3


def full_check(oracle, A, B, tau):
    from cuspamm_b200 import SpammPlan

    n = A.shape[0]
    C_ref, S, nA, nB, counts = oracle.spamm(A, B, tau, want_maps=True)
    with SpammPlan(n, A.shape[1], B.shape[1]) as p:
        p.upload(A, B)
        p.run(tau)
        p.sync()
        C = p.download_c()
        got_counts, got_s = p.counts()
        assert np.array_equal(p.norm_a().view(np.uint32), nA.view(np.uint32))
        assert np.array_equal(p.norm_b().view(np.uint32), nB.view(np.uint32))
    assert got_s == S and np.array_equal(got_counts, counts)
    err = rel_fro(C, C_ref)
    assert err <= C_TOL, err
    return S, err


@pytest.mark.parametrize("tau", [1e-10, 1e-6, 1e-4, 1e-2])
def test_config2_exponential_decay_sweep(oracle, tau):
    """Exponential decay at N=4096: a_ij = +-exp(-0.1|i-j|), independent seeds, the sweep's non-zero thresholds."""
    from cuspamm_b200 import gen_signed_exp

    n = 4096
    A, B = gen_signed_exp(0.1, 1, n, n), gen_signed_exp(0.1, 2, n, n)
    S, err = full_check(oracle, A, B, tau)
    assert 0 < S < (n // 32) ** 3 // 20
    assert err < 1e-5


def test_config2_dense_limit_tau_zero():
    """tau = 0 keeps every product (0 >= 0 included): C is the product of the half-rounded inputs."""
    import torch

    from cuspamm_b200 import SpammPlan, gen_signed_exp

    n = 4096
    A, B = gen_signed_exp(0.1, 1, n, n), gen_signed_exp(0.1, 2, n, n)
    with SpammPlan(n, n, n) as p:
        C, st = p.multiply(A, B, 0.0)
    assert st["survivors"] == (n // 32) ** 3
    torch.backends.cuda.matmul.allow_tf32 = False
    ref = (torch.from_numpy(A).cuda().half().float() @ torch.from_numpy(B).cuda().half().float()).cpu().numpy()
    assert rel_fro(C, ref) < 1e-5


def test_config3_algebraic_decay(oracle):
    """Algebraic decay: a_ij = u_ij/(|i-j|^2+1), u in [-1,1); exact check at N=4096."""
    from cuspamm_b200 import gen_uniform_alg

    n = 4096
    A, B = gen_uniform_alg(3, n, n), gen_uniform_alg(4, n, n)
    S, err = full_check(oracle, A, B, 1e-6)
    assert err < 1e-5


def test_config4_lattice(oracle):
    """Density-matrix surrogate on a 16^3 lattice (N=4096): symmetric, list lengths spread over a wide range."""
    from cuspamm_b200 import gen_lattice

    A = gen_lattice(16, 7)
    assert np.array_equal(A, A.T)
    S, err = full_check(oracle, A, A.copy(), 1e-8)
    assert err < 1e-5


def test_full_size_properties_n16384(oracle):
    """N=16384 (the headline size): counts against the checker's count on the library's own (bit-checked) norm maps,
    one row block against the checker, two half-height plans against the full one, and a repeat of the run."""
    from cuspamm_b200 import SpammPlan, gen_signed_exp

    n, tau = 16384, 1e-6
    A, B = gen_signed_exp(0.1, 1, n, n), gen_signed_exp(0.1, 2, n, n)
    T = n // 32
    with SpammPlan(n, n, n) as p:
        p.upload(A, B)
        p.run(tau)
        p.sync()
        C = p.download_c()
        nA, nB = p.norm_a(), p.norm_b()
        counts, S = p.counts()
        p.run(tau)
        p.sync()
        assert np.array_equal(p.download_c(), C)            # same lists, same order of accumulation
    # norm maps: two tile rows bit for bit (the full map is checked at smaller sizes)
    assert np.array_equal(nA[40:42].view(np.uint32), oracle.norm_map(A[40 * 32:42 * 32]).view(np.uint32))
    assert np.array_equal(nB[500:502].view(np.uint32), oracle.norm_map(B[500 * 32:502 * 32]).view(np.uint32))
    c_counts, _, _ = oracle.lists(nA, nB, tau)
    assert np.array_equal(counts, c_counts) and S == int(c_counts.sum())
    assert S == 55344                                        # recorded with the first verified run of this workload
    # a block of 8 tile rows against the checker
    C_blk, S_blk = oracle.spamm(A, B, tau, row_begin=200, row_count=8)
    assert S_blk == int(counts[200:208].sum())
    assert rel_fro(C[200 * 32:208 * 32], C_blk) <= C_TOL
    # everything outside the band of surviving tiles is exactly zero
    Ct = np.abs(C).reshape(T, 32, T, 32).max(axis=(1, 3))
    assert not Ct[counts == 0].any()
    # the reference's row split: two plans, each half of the tile rows, reproduce the full C
    parts = []
    for b0 in (0, T // 2):
        with SpammPlan(n, n, n, b0, T // 2) as q:
            q.upload(np.ascontiguousarray(A[b0 * 32:(b0 + T // 2) * 32]), B)
            q.run(tau)
            q.sync()
            parts.append(q.download_c())
    assert rel_fro(np.vstack(parts), C) < 1e-6


def test_config5_dense_uniform_rows_sample():
    """Dense uniform matrices, tau=0, at N=8192: every product executed, rows checked against a float product."""
    import torch

    from cuspamm_b200 import SpammPlan, gen_uniform

    n = 8192
    A, B = gen_uniform(5, n, n), gen_uniform(6, n, n)
    with SpammPlan(n, n, n) as p:
        C, st = p.multiply(A, B, 0.0)
    assert st["survivors"] == (n // 32) ** 3
    torch.backends.cuda.matmul.allow_tf32 = False
    Bh = torch.from_numpy(B).cuda().half().float()
    for r0 in (0, 4000, 8192 - 256):
        ref = (torch.from_numpy(A[r0:r0 + 256]).cuda().half().float() @ Bh).cpu().numpy()
        assert rel_fro(C[r0:r0 + 256], ref) < 1e-5


def test_error_norms_against_dense_product(oracle):
    """The reference's comparator figures (tool.cu:6-24): ||dense - spamm||, ||dense||, ||spamm|| on the GPU, with the
    dense product made by the same plan at tau = 0."""
    import torch

    from cuspamm_b200 import BUF_C, SpammPlan, gen_signed_exp

    n = 2048
    A, B = gen_signed_exp(0.1, 1, n, n), gen_signed_exp(0.1, 2, n, n)
    with SpammPlan(n, n, n) as p:
        p.upload(A, B)
        p.run(0.0)
        p.sync()
        dense = p.as_tensor(BUF_C).clone()
        p.run(1e-2)
        p.sync()
        e, r, o = p.error_norms(dense.data_ptr())
        C = p.download_c()
    D = dense.cpu().numpy().astype(np.float64)
    assert abs(r - np.linalg.norm(D)) <= 1e-9 * r
    assert abs(o - np.linalg.norm(C.astype(np.float64))) <= 1e-9 * o
    assert abs(e - np.linalg.norm(D - C)) <= 1e-9 * max(e, 1e-30) + 1e-12
    assert 0 < e / r < 0.1                     # tau = 1e-2 drops little of an exponentially decaying product


def test_cnn_im2col_shape_with_padding(oracle):
    """The reference's CNN use case (para.h:19-22): a 64x576 weight matrix times a 576x102400 im2col matrix; with
    sizes that are not multiples of 32 padded with zeros as main.h:54-56 pads them (here 60x570 and 570x4000)."""
    from cuspamm_b200 import SpammPlan, pad_to_tiles

    rng = np.random.default_rng(9)
    W = (rng.standard_normal((64, 576)) * np.exp(-4 * rng.random((64, 576)))).astype(np.float32)
    X = (rng.standard_normal((576, 102400 // 8)) * np.exp(-4 * rng.random((576, 102400 // 8)))).astype(np.float32)
    tau = 127.0                                # about the median norm product of these matrices
    with SpammPlan(64, 576, X.shape[1]) as p:
        C, st = p.multiply(W, X, tau)
    C_ref, S = oracle.spamm(W, X, tau)
    assert st["survivors"] == S and 0 < S < st["tile_products"]
    assert rel_fro(C, C_ref) <= C_TOL
    Wp, Xp = pad_to_tiles(W[:60, :570]), pad_to_tiles(X[:570, :4000])
    assert Wp.shape == (64, 576) and Xp.shape == (576, 4000)
    with SpammPlan(*Wp.shape, Xp.shape[1]) as p:
        Cp, st = p.multiply(Wp, Xp, 0.0)
    dense = W[:60, :570].astype(np.float16).astype(np.float64) @ X[:570, :4000].astype(np.float16).astype(np.float64)
    assert rel_fro(Cp[:60, :4000], dense) < 1e-5
    assert not Cp[60:].any()


def test_cnn_im2col_full_shape(oracle):
    """The reference's CNN case at its full size (para.h:19-22): 64 x 576 weights times a 576 x 102400 im2col matrix
    (synthetic stand-ins for the missing data files, same shapes)."""
    from cuspamm_b200 import SpammPlan

    rng = np.random.default_rng(10)
    W = (rng.standard_normal((64, 576)) * np.exp(-4 * rng.random((64, 576)))).astype(np.float32)
    X = (rng.standard_normal((576, 102400), dtype=np.float32) *
         np.exp(-4 * rng.random((576, 102400), dtype=np.float32))).astype(np.float32)
    tau = 127.0
    C_ref, S, nA, nB, counts = oracle.spamm(W, X, tau, want_maps=True)
    with SpammPlan(64, 576, 102400) as p:
        C, st = p.multiply(W, X, tau)
        assert np.array_equal(p.norm_b().view(np.uint32), nB.view(np.uint32))
        got_counts, _ = p.counts()
    assert st["survivors"] == S and 0 < S < st["tile_products"]
    assert np.array_equal(got_counts, counts)
    assert rel_fro(C, C_ref) <= C_TOL


def test_command_line_driver(oracle):
    """cuspamm_b200/spamm_main, the C++ caller of the boundary with the shape of the reference's `main`: its default
    run (2048^3, c/(|i-j|^v+1) with c=v=0.1, Norm=1.548969; para.h:2,6-8,14) keeps as many products as the checker, and
    the all-ones input keeps all of them at the threshold 1024."""
    import re
    import subprocess

    from cuspamm_b200 import build, gen_decay_alg

    exe = build.build_driver()
    A = gen_decay_alg(0.1, 0.1, 2048, 2048)
    _, S = oracle.spamm(A, A.copy(), 1.548969)
    r = subprocess.run([str(exe), "--iters", "3", "--warmup", "1"], stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                       text=True, timeout=300)
    assert r.returncode == 0, r.stdout
    assert int(re.search(r"valid mul=(\d+)", r.stdout).group(1)) == S
    assert re.search(r"SpAMM time=\d", r.stdout)
    r = subprocess.run([str(exe), "--n", "250", "--matrix", "ones", "--tau", "1000", "--iters", "2", "--warmup", "1"],
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300)
    assert r.returncode == 0, r.stdout
    # 250 = 7 full tiles + a 26-wide rest: the products of full tiles (32*32 = 1024) pass 1000, those with a
    # partial tile (32*sqrt(32*26) = 923, or 26*32 = 832) do not
    assert int(re.search(r"valid mul=(\d+)", r.stdout).group(1)) == 7 ** 3
