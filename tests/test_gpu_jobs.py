"""The job-list matvec (launch_qmatvec_batch: several projections in one persistent launch) against
the CPU oracle and against the single-matrix launcher, through the C ABI.  Needs a B200.

Bars as for the single matvec: fp32 outputs within 1e-3 relative / 1e-4 absolute of the oracle;
bit-identical across reruns."""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

REL_TOL, ABS_TOL = 1e-3, 1e-4


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.fail("these tests need a CUDA device")
    from nates_recipe_rs_b200 import quant_ops
    return quant_ops


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def assert_close(got, want, what=""):
    err = np.abs(got.astype(np.float64) - want.astype(np.float64))
    bound = ABS_TOL + REL_TOL * np.abs(want.astype(np.float64))
    bad = err > bound
    assert not bad.any(), f"{what}: {bad.sum()} of {bad.size} outside tolerance, max err {err.max():.3e}"


def make_job(qtype, n, k, m, seed):
    w = oracle.quantize(qtype, oracle.fill_normal(n * k, seed, 0.02).reshape(n, k))
    x = oracle.fill_normal(m * k, seed + 1000, 1.0).reshape(m, k)
    xq = oracle.quantize(oracle.Q8_1, x)
    return w, xq, oracle.matvec(qtype, w, xq, k)


def run_list(ops, specs, m, seed=1):
    """specs: [(qtype, n, k)]; returns (got list, want list)."""
    jobs = ops.MatvecJobs()
    outs, wants = [], []
    for i, (qtype, n, k) in enumerate(specs):
        w, xq, want = make_job(qtype, n, k, m, seed + 17 * i)
        y = torch.full((m, n), float("nan"), device="cuda")
        jobs.add(qtype, dev(w), dev(xq), y, n, k)
        outs.append(y)
        wants.append(want)
    ops.gpu_qmatvec_batch_into(jobs, m)
    torch.cuda.synchronize()
    ops.check_launch()
    return [y.cpu().numpy() for y in outs], wants


Q8, Q4, Q6 = oracle.Q8_0, oracle.Q4_K, oracle.Q6_K

LISTS = [
    # one job; fewer rows than CTAs; a row count that is no multiple of anything
    [(Q4, 1, 256)], [(Q4, 37, 512)], [(Q6, 150, 1024)], [(Q8, 149, 256)],
    # mixed types and K in one list, short and long jobs alternating (stages of different jobs share the ring)
    [(Q4, 300, 1024), (Q6, 7, 2048), (Q8, 513, 4096), (Q4, 1000, 4096), (Q6, 257, 4096)],
    # the FFN shapes of the decode benchmark at reduced width, then a Q8_0 K that is 2-byte aligned only
    [(Q4, 1792, 4096), (Q4, 1792, 4096), (Q4, 512, 14336), (Q6, 512, 14336)],
    [(Q8, 333, 4224), (Q6, 91, 14336), (Q4, 40, 28672)],
    # many tiny jobs: activations of the next job land while the current one has a single stage
    [(Q4, 5 + 3 * i, 256 * (1 + i % 3)) for i in range(12)],
]


@pytest.mark.parametrize("m", [1, 2])
@pytest.mark.parametrize("specs", LISTS, ids=[f"list{i}" for i in range(len(LISTS))])
def test_job_list_matches_oracle(ops, specs, m):
    got, want = run_list(ops, specs, m)
    for i, (g, w) in enumerate(zip(got, want)):
        assert not np.isnan(g).any(), f"job {i}: rows left unwritten"
        assert_close(g, w, f"job {i} {specs[i]}")


@pytest.mark.parametrize("warps", [8, 12, 16, 21, 24])
def test_job_list_other_warp_counts(ops, warps):
    """The split of a CTA's warps into K slices and row groups differs per job and with the warp count
    (tunable "jobs_warps"); warps without a share in a job still take part in every hand-over."""
    from nates_recipe_rs_b200._lib import check, lib
    check(lib().qmm_tune(b"jobs_warps", warps), "qmm_tune")
    try:
        for specs in (LISTS[4], LISTS[6], LISTS[7]):
            for rep in range(3):   # timing-dependent faults would differ between repetitions
                got, want = run_list(ops, specs, 1, seed=11 + rep)
                for i, (g, w) in enumerate(zip(got, want)):
                    assert_close(g, w, f"warps {warps} rep {rep} job {i} {specs[i]}")
    finally:
        check(lib().qmm_tune(b"jobs_warps", 14), "qmm_tune")


def test_job_list_longer_than_one_launch_and_rerun_bit_identical(ops):
    specs = [((Q4, Q6, Q8)[i % 3], 64 + i, 512) for i in range(45)]   # more than the 40 jobs one launch takes
    a, want = run_list(ops, specs, 1, seed=5)
    b, _ = run_list(ops, specs, 1, seed=5)
    for i in range(len(specs)):
        assert_close(a[i], want[i], f"job {i}")
        assert np.array_equal(a[i].view(np.uint32), b[i].view(np.uint32)), f"job {i}: rerun differs"


def test_job_list_equals_single_launches_on_ffn_shapes(ops):
    """Full-size FFN shapes of the decode benchmark: same arithmetic and fold order as the single-matrix
    kernel, so the outputs are equal bit for bit when both use the same K split."""
    m = 1
    specs = [(Q4, 14336, 4096), (Q4, 14336, 4096), (Q4, 4096, 14336), (Q6, 4096, 14336)]
    jobs = ops.MatvecJobs()
    pairs = []
    for i, (qtype, n, k) in enumerate(specs):
        g = torch.Generator(device="cuda").manual_seed(40 + i)
        w = ops.gpu_quantize_weights(qtype, torch.randn(n, k, device="cuda", generator=g) * 0.02)
        xq = ops.gpu_quantize_q8_1(torch.randn(m, k, device="cuda", generator=g))
        y = torch.zeros(m, n, device="cuda")
        jobs.add(qtype, w, xq, y, n, k)
        pairs.append((qtype, w, xq, y, n, k))
    ops.gpu_qmatvec_batch_into(jobs, m)
    for qtype, w, xq, y, n, k in pairs:
        ref = ops.gpu_qmatvec(qtype, w, xq, m, n, k)
        assert torch.allclose(y, ref, rtol=REL_TOL, atol=ABS_TOL), (qtype, n, k, float((y - ref).abs().max()))
    # a row sample against the oracle
    qtype, w, xq, y, n, k = pairs[3]
    rows = np.arange(0, n, 97)
    wn = w.cpu().numpy().reshape(n, -1)[rows]
    want = oracle.matvec(qtype, wn, xq.cpu().numpy(), k)
    assert_close(y.cpu().numpy()[:, rows], want, "Q6_K down rows")
    ops.check_launch()


def test_job_list_device_side_selector(ops):
    """A job whose matrix is chosen on the device: w + select[0] * stride (an expert picked by a router)."""
    m, n, k, experts = 1, 200, 1024, 5
    rb = oracle.row_bytes(Q4, k)
    bank = [oracle.quantize(Q4, oracle.fill_normal(n * k, 300 + e, 0.02).reshape(n, k)) for e in range(experts)]
    bank_d = dev(np.stack(bank))
    x = oracle.fill_normal(k, 9, 1.0)
    xq = oracle.quantize(oracle.Q8_1, x)
    xq_d = dev(xq)
    picks = [3, 0, 4]
    sel = [torch.tensor([e], dtype=torch.int32, device="cuda") for e in picks]
    outs = [torch.zeros(m, n, device="cuda") for _ in picks]
    jobs = ops.MatvecJobs()
    for s, y in zip(sel, outs):
        jobs.add(Q4, bank_d, xq_d, y, n, k, select=s, select_stride_bytes=n * rb)
    ops.gpu_qmatvec_batch_into(jobs, m)
    torch.cuda.synchronize()
    for e, y in zip(picks, outs):
        assert_close(y.cpu().numpy(), oracle.matvec(Q4, bank[e], xq, k), f"expert {e}")
    ops.check_launch()


def test_job_list_falls_back_and_rejects(ops):
    from nates_recipe_rs_b200._lib import lib, MatvecJob
    # m = 5 is outside the persistent kernel: the launcher runs one launch per job, same results
    got, want = run_list(ops, [(Q4, 130, 4096), (Q6, 70, 2048)], 5)
    for g, w in zip(got, want):
        assert_close(g, w, "fallback")
    L = lib()
    assert L.launch_qmatvec_batch(None, 1, 1, None) == -1
    j = (MatvecJob * 1)(MatvecJob(Q4, 8, 100, 16, 16, 16, 0, None, 0, 0))
    assert L.launch_qmatvec_batch(j, 1, 1, None) == -2
    j = (MatvecJob * 1)(MatvecJob(99, 8, 256, 16, 16, 16, 0, None, 0, 0))
    assert L.launch_qmatvec_batch(j, 1, 1, None) == -5
    j = (MatvecJob * 1)(MatvecJob(Q4, 8, 256, 16, 16, 16, 0, 16, 24, 0))   # selector stride not a multiple of 16
    assert L.launch_qmatvec_batch(j, 1, 1, None) == -4


def test_tp_exchange_with_one_rank_equals_plain_launches(ops):
    """The tensor-parallel entry points with a world of one rank: the outputs travel through the exchange
    area (push, poll, sum of one term) and must equal the plain launchers bit for bit, exchange after
    exchange (the two buffers alternate; the sequence counter advances on the device)."""
    import ctypes as C
    from nates_recipe_rs_b200._lib import check, lib
    L = lib()
    comm = C.c_void_p()
    check(L.qmm_tp_comm_create(0, 1, 16 * 4096, C.byref(comm)), "qmm_tp_comm_create")
    stream = torch.cuda.current_stream().cuda_stream
    try:
        for rep, (qtype, n, k, m) in enumerate([(Q4, 4096, 1024, 1), (Q6, 1000, 2048, 2), (Q4, 4096, 2048, 16), (Q8, 333, 512, 3), (Q6, 512, 4096, 7)]):
            g = torch.Generator(device="cuda").manual_seed(70 + rep)
            w = ops.gpu_quantize_weights(qtype, torch.randn(n, k, device="cuda", generator=g) * 0.02)
            xq = ops.gpu_quantize_q8_1(torch.randn(m, k, device="cuda", generator=g))
            y = torch.full((m, n), float("nan"), device="cuda")
            check(L.launch_qmatvec_tp(comm, qtype, w.data_ptr(), xq.data_ptr(), y.data_ptr(), m, n, k, stream), "launch_qmatvec_tp")
            assert torch.equal(y, ops.gpu_qmatvec(qtype, w, xq, m, n, k)), (rep, qtype, n, k, m)
        # a job list with summed and local jobs
        jobs = ops.MatvecJobs()
        pairs = []
        for i, (qtype, n, k, summed) in enumerate([(Q4, 1024, 1024, False), (Q4, 2048, 1792, True), (Q6, 512, 1792, True), (Q4, 4096, 512, True)]):
            g = torch.Generator(device="cuda").manual_seed(90 + i)
            w = ops.gpu_quantize_weights(qtype, torch.randn(n, k, device="cuda", generator=g) * 0.02)
            xq = ops.gpu_quantize_q8_1(torch.randn(1, k, device="cuda", generator=g))
            y = torch.full((1, n), float("nan"), device="cuda")
            jobs.add(qtype, w, xq, y, n, k, tp_sum=summed)
            pairs.append((qtype, w, xq, y, n, k))
        arr = jobs.array()
        for _ in range(3):
            check(L.launch_qmatvec_batch_tp(comm, arr, len(jobs), 1, stream), "launch_qmatvec_batch_tp")
        for qtype, w, xq, y, n, k in pairs:
            assert torch.allclose(y, ops.gpu_qmatvec(qtype, w, xq, 1, n, k), rtol=REL_TOL, atol=ABS_TOL)
        ops.check_launch()
        # too large for the exchange area
        big = torch.zeros(8, device="cuda")
        assert L.launch_qmatvec_tp(comm, Q4, big.data_ptr(), big.data_ptr(), big.data_ptr(), 32, 4096, 256, stream) == -7
    finally:
        check(L.qmm_tp_comm_destroy(comm), "qmm_tp_comm_destroy")


@pytest.mark.parametrize("m", [1, 2])
@pytest.mark.parametrize("k,with_add", [(4096, True), (1024, False), (8192, True)])
def test_norm_built_inside_the_job_launch(ops, m, k, with_add):
    """launch_norm_qmatvec_batch: residual add + RMSNorm + Q8_1 inside the launch, shared by the jobs."""
    x = oracle.fill_normal(m * k, 1, 1.3).reshape(m, k)
    add = oracle.fill_normal(m * k, 2, 0.6).reshape(m, k) if with_add else None
    gamma = oracle.fill_normal(k, 3, 0.1) + np.float32(1.0)
    xs = x + add if with_add else x
    xq = oracle.quantize(oracle.Q8_1, oracle.rmsnorm(xs, gamma, 1e-6))
    specs = [(Q4, 700, k), (Q6, 260, k), (Q8, 129, k)]
    jobs = ops.MatvecJobs()
    outs, wants = [], []
    for i, (qtype, n, _) in enumerate(specs):
        w = oracle.quantize(qtype, oracle.fill_normal(n * k, 20 + i, 0.02).reshape(n, k))
        y = torch.full((m, n), float("nan"), device="cuda")
        jobs.add(qtype, dev(w), None, y, n, k)
        outs.append(y)
        wants.append(oracle.matvec(qtype, w, xq, k))
    x_out = torch.full((m, k), float("nan"), device="cuda") if with_add else None
    ops.gpu_norm_qmatvec_batch_into(dev(x), dev(add) if with_add else None, dev(gamma), x_out, 1e-6, jobs, m)
    torch.cuda.synchronize()
    ops.check_launch()
    if with_add:
        assert np.array_equal(x_out.cpu().numpy(), xs), "updated residual"
    for i, (y, want) in enumerate(zip(outs, wants)):
        # the sum of squares is added in another order than on the host: an activation code may differ by one
        err = np.abs(y.cpu().numpy() - want)
        assert (err <= 1e-4 + 1e-3 * np.abs(want) + 2e-3 * np.abs(want).max()).all(), (i, float(err.max()))
        assert np.median(err / (np.abs(want) + 1e-6)) < 1e-4


@pytest.mark.parametrize("act", [0, 1])
def test_gated_activation_built_inside_the_job_launch(ops, act):
    m, k, n = 2, 3584, 1000
    gu = oracle.fill_normal(m * 2 * k, 5, 1.5).reshape(m, 2 * k)
    fn = oracle.gelu_mul if act == 0 else oracle.silu_mul
    xq = oracle.quantize(oracle.Q8_1, fn(gu[:, :k].copy(), gu[:, k:].copy()))
    w = oracle.quantize(Q6, oracle.fill_normal(n * k, 6, 0.02).reshape(n, k))
    y = torch.full((m, n), float("nan"), device="cuda")
    jobs = ops.MatvecJobs().add(Q6, dev(w), None, y, n, k)
    ops.gpu_glu_qmatvec_batch_into(dev(gu), act, jobs, m)
    torch.cuda.synchronize()
    ops.check_launch()
    want = oracle.matvec(Q6, w, xq, k)
    err = np.abs(y.cpu().numpy() - want)
    assert (err <= 1e-4 + 1e-3 * np.abs(want) + 2e-3 * np.abs(want).max()).all(), float(err.max())
