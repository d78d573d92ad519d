"""The workspace-size queries of the C-ABI are pure functions of the shapes:
checked here without a GPU against the layouts the kernels use."""

from hc_b200 import capi


def _round_up(value, step):
    return -(-value // step) * step


def test_dequant_gemm_workspaces():
    lib = capi.load_kernels()
    # The whole converted matrix, rows padded to 16 columns.
    assert lib.hcGemmW8A16WorkspaceBytes(8192, 8192) == 8192 * 8192 * 2
    assert lib.hcGemmW8A16WorkspaceBytes(264, 520) == 272 * 520 * 2
    assert lib.hcGemmW8A16WorkspaceBytes(0, 5) == 0
    # The banded form: a ring of three bands of 1024 columns and two counters per band.
    assert lib.hcGemmW8A16BandedBytes(8192, 8192) == 3 * 8192 * 1024 * 2 + 256
    assert lib.hcGemmW8A16BandedBytes(4368, 128) == 3 * 128 * 1024 * 2 + 256  # five bands
    assert lib.hcGemmW8A16BandedBytes(40000, 64) == 3 * 64 * 1024 * 2 + 512   # forty bands
    assert lib.hcGemmW8A16BandedBytes(0, 64) == 0


def test_convolution_workspace_covers_both_layouts():
    lib = capi.load_kernels()
    for n, c, h, w, nf, hf, wf in [(32, 64, 56, 56, 64, 3, 3), (2, 40, 16, 70, 24, 3, 3),
                                   (1, 1, 5, 5, 1, 1, 1), (5, 7, 9, 40, 200, 3, 3)]:
        need = lib.hcConvF32TensorWorkspaceBytes(n, c, h, w, nf, hf, wf)
        k = c * hf * wf
        # Gathering kernels: the filters as [NF, K rounded up to 4] (hi, lo), x as (hi, lo) pairs.
        gathered = 2 * _round_up(nf * _round_up(k, 4) * 4, 1024) + _round_up(n * c * h * w * 8, 1024)
        # TMA kernels: channels rounded up to 32 in the filters [NF, taps * Cp] and in the image
        # [N, H * W, Cp], hi and lo parts each.
        cp = _round_up(c, 32)
        by_tma = 2 * _round_up(nf * hf * wf * cp * 4, 1024) + 2 * _round_up(n * h * w * cp * 4, 1024)
        assert need == max(gathered, by_tma)
        assert need % 1024 == 0
    assert lib.hcConvF32TensorWorkspaceBytes(0, 3, 8, 8, 4, 3, 3) == 0


def test_float32_gemm_workspace():
    lib = capi.load_kernels()
    m, n, k = 300, 200, 101  # K rounded up to 4 in both split operands
    assert lib.hcGemmF32TensorWorkspaceBytes(m, n, k) == (
        2 * _round_up(m * 104 * 4, 1024) + 2 * _round_up(n * 104 * 4, 1024))
