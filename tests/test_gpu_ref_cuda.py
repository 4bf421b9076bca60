"""The reference's own CUDA backend on this GPU (compiled from the reference sources into
oracle/_ref, sm_100): used to pin the oracle's restatement of the CUDA RMSNorm and as a sanity
check of the same-box baseline that bench.py times. Skipped where oracle/_ref is not built."""
import numpy as np
import pytest

from tensorlib_b200 import synth

pytestmark = pytest.mark.gpu


def ulp_distance(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """Distance in fp16 steps between two arrays of the same sign pattern (monotone integer map)."""
    def key(v):
        u = np.ascontiguousarray(v).view(np.uint16).astype(np.int32)
        return np.where(u & 0x8000, -(u & 0x7FFF), u)
    return np.abs(key(a) - key(b))


def test_oracle_cuda_route_rmsnorm_matches_the_reference_kernel(tl, oracle, ref):
    """rms_norm_kernel_v1 (tensorLib/src/device/cuda/rms_norm.cu:138-167) against its restatement:
    at most one fp16 step apart (the order of the warp-level sum is not documented, and the device's
    half division may differ from the correctly rounded quotient in the last place)."""
    assert ref.cuda_device_count() >= 1
    for (T, D, std) in ((1, 4096, 1.0), (5, 4096, 0.3), (3, 288, 1.0), (2, 11008, 2.0)):
        x = synth.normal_f16(61, T + D, T * D, std).reshape(T, D)
        w = synth.normal_f16(61, 7, D, 1.0)
        got, want = ref.cuda_rms_norm(x, w), oracle.rmsnorm_cuda_route(x, w)
        d = ulp_distance(got, want)
        assert d.max() <= 1, (T, D, int(d.max()))
        print(f"rms_norm {T}x{D}: {(d == 0).mean():.4f} of the values bit-equal, the rest one step apart")


def test_reference_cuda_matmul_route_agrees_with_its_cpu_route(tl, oracle, ref):
    """CUDA<half>::matmul2d (gemv_v6 for K in {4096, 11008}, gemv_v4 otherwise, cuBLAS for M > 1;
    gemm.cu:153-172) against the CPU oracle, within the matmul tolerance. N is kept a multiple of 4
    and K a multiple of 8: gemv_v6 has no bounds check (gemv.cu:379-434)."""
    for (M, N, K) in ((1, 512, 4096), (1, 256, 11008), (1, 64, 288), (16, 256, 1024)):
        A = synth.normal_f16(62, M, M * K, 1.0).reshape(M, K)
        W = synth.normal_f16(62, 2, N * K, 0.02).reshape(N, K)
        got, _ = ref.cuda_matmul2d(A, W)
        want = oracle.matmul2d(A, W).astype(np.float64)
        scale = np.sqrt((want * want).mean(axis=-1, keepdims=True)) + 1e-30
        rel = (np.abs(got.astype(np.float64) - want) / np.maximum(np.abs(want), scale)).max()
        assert rel <= 1e-2, (M, N, K, rel)
