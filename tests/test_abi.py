"""The C-ABI library builds, loads and exports every symbol include/hawk_b200.h declares; its
host-side argument validation answers without touching a GPU.  CPU only."""
import ctypes
import os
import re

import pytest

from conftest import ROOT

import hawk_b200._lib as L


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "hawk_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(hawk_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = L.load()
    names = _declared_symbols()
    assert "hawk_scan_fwd" in names and "hawk_conv1d_bwd" in names
    for n in names:
        assert hasattr(lib, n), n
    assert sorted(L.SIGNATURES) == names  # the ctypes table covers the header one to one
    assert lib.hawk_version() == L.ABI_VERSION


def test_strerror_is_total():
    lib = L.load()
    assert lib.hawk_strerror(0) == b"ok"
    for code in range(-8, 0):
        assert len(lib.hawk_strerror(code)) > 3
    assert b"unknown" in lib.hawk_strerror(-99)


def test_scan_argument_validation_needs_no_gpu():
    lib = L.load()
    p = ctypes.c_void_p(4096)  # never dereferenced: validation fails first
    assert lib.hawk_scan_fwd(None, p, p, p, None, None, p, 1, 8, 64, L.HAWK_BF16, None) == -1      # NULL
    assert lib.hawk_scan_fwd(p, p, p, p, None, None, p, 1, 8, 96, L.HAWK_BF16, None) == -2         # D % 64
    assert lib.hawk_scan_fwd(p, p, p, p, None, None, p, 1, 0, 64, L.HAWK_BF16, None) == -2         # T < 1
    assert lib.hawk_scan_fwd(p, p, p, p, None, None, p, 1, 8, 64, 7, None) == -3                   # dtype
    assert lib.hawk_scan_fwd(ctypes.c_void_p(4098), p, p, p, None, None, p, 1, 8, 64, L.HAWK_BF16, None) == -4
    assert lib.hawk_scan_fwd(p, p, p, p, None, ctypes.c_void_p(4100), p, 1, 8, 64, L.HAWK_BF16, None) == -4  # gate_bias
    assert lib.hawk_scan_bwd_workspace_bytes(8, 2048) == 3 * 8 * 2048 * 4
    # x gx ga lam | h0 gate_bias | h go dx dgx dga dlam | dh0 dgate_bias
    args = [p] * 4 + [None, None] + [p] * 6 + [None, None]
    assert lib.hawk_scan_bwd(*args, p, 16, 8, 16, 2048, L.HAWK_BF16, None) == -5             # workspace too small
    one_plane = 8 * 2048 * 4  # enough without the gate-bias gradients, too small with them
    args = [p] * 4 + [None, p] + [p] * 6 + [None, p]
    assert lib.hawk_scan_bwd(*args, p, one_plane, 8, 16, 2048, L.HAWK_BF16, None) == -5


def test_conv_argument_validation_needs_no_gpu():
    lib = L.load()
    p = ctypes.c_void_p(4096)
    assert lib.hawk_conv1d_fwd(p, 0, 64, p, p, p, 1, 8, 64, 5, 1, 1, None) == -7   # width 5 unsupported
    assert lib.hawk_conv1d_fwd(p, 0, 64, p, p, p, 1, 8, 60, 4, 1, 1, None) == -2   # D % 8
    assert lib.hawk_conv1d_fwd(p, 0, 68, p, p, p, 1, 8, 64, 4, 1, 1, None) == -4   # row stride % 8
    assert lib.hawk_conv1d_bwd_workspace_bytes(8, 4096, 2048, 4) == 8 * 8 * 5 * 2048 * 4  # 64-row tiles, 8 per CTA


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(L, "_lib", None)
    monkeypatch.setattr(L, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no fallback"):
        L.load()


def test_ops_refuse_cpu_tensors():
    import torch
    from hawk_b200 import fused_linear_scan
    x = torch.zeros(1, 4, 64)
    with pytest.raises(RuntimeError, match="CUDA"):
        fused_linear_scan(x, x, x, torch.zeros(64))


def test_glue_ce_and_decode_argument_validation_needs_no_gpu():
    lib = L.load()
    p = ctypes.c_void_p(4096)
    # gelu_mul: width and pitches in multiples of 8, pitch >= width
    assert lib.hawk_gelu_mul_fwd(p, 64, p, 64, p, 64, 4, 60, 1, None) == -2
    assert lib.hawk_gelu_mul_fwd(p, 32, p, 64, p, 64, 4, 64, 1, None) == -2
    assert lib.hawk_gelu_mul_fwd(p, 68, p, 64, p, 64, 4, 64, 1, None) == -4
    assert lib.hawk_gelu_mul_bwd(p, 64, p, 64, p, 64, None, 64, p, 64, 4, 64, 1, None) == -1
    # rms_norm: H % 4, backward H <= 4096, workspace
    assert lib.hawk_rms_norm_fwd(p, p, p, p, 4, 66, 1e-6, 0, 1, None) == -2
    assert lib.hawk_rms_norm_bwd_workspace_bytes(2048) == 296 * 2048 * 4
    assert lib.hawk_rms_norm_bwd(p, p, p, p, p, p, p, 1 << 30, 4, 8192, 0, 1, None) == -2
    assert lib.hawk_rms_norm_bwd(p, p, p, p, p, p, p, 16, 4, 2048, 0, 1, None) == -5
    assert lib.hawk_add_rms_norm_fwd(p, None, p, p, p, p, 4, 64, 1e-6, 0, 1, None) == -1
    # linear cross-entropy: H % 8, workspace size, alignment
    assert lib.hawk_linear_ce_fwd_bwd(p, p, p, p, p, p, p, 1 << 40, 16, 60, 100, 0, p, None) == -2
    need = lib.hawk_linear_ce_workspace_bytes(16, 64, 100)
    assert need > 16 * 100 * 2 * 2
    assert lib.hawk_linear_ce_fwd_bwd(p, p, p, p, p, p, p, need - 1, 16, 64, 100, 0, p, None) == -5
    assert lib.hawk_linear_ce_fwd_bwd(p, p, p, p, p, p, ctypes.c_void_p(4096 + 64), need, 16, 64, 100, 0, p, None) == -4
    # decode steps
    assert lib.hawk_decode_conv_step(p, 64, p, p, p, p, 2, 60, 4, 1, 1, None) == -2
    assert lib.hawk_decode_conv_step(p, 64, p, p, p, p, 2, 64, 5, 1, 1, None) == -7
    assert lib.hawk_decode_rglru_step(p, p, p, p, None, p, 2, 64, 1, 1, None) == -1
    # the no-allocation backward refuses what its built-in scratch cannot hold
    assert lib.hawk_scan_bwd_noalloc(p, p, p, p, None, p, p, p, p, p, p, None, 129, 8, 2048, 1, None) == -9


def test_cast_and_adamw_argument_validation_needs_no_gpu():
    lib = L.load()
    p = ctypes.c_void_p(4096)
    assert lib.hawk_cast_f32_bf16(None, p, 8, None) == -1
    assert lib.hawk_cast_f32_bf16(p, p, 0, None) == -2
    assert lib.hawk_cast_f32_bf16(ctypes.c_void_p(4100), p, 8, None) == -4
    adam = (1e-3, 0.9, 0.999, 1e-8, 0.1)
    assert lib.hawk_adamw_step(p, None, p, p, None, 8, *adam, 1, None) == -1      # gradient missing
    assert lib.hawk_adamw_step(p, p, p, p, None, 0, *adam, 1, None) == -2         # n < 1
    assert lib.hawk_adamw_step(p, p, p, p, None, 8, *adam, 0, None) == -2         # step counts from 1
    assert lib.hawk_adamw_step(ctypes.c_void_p(4098), p, p, p, None, 8, *adam, 1, None) == -4


def test_decode_block_step_argument_validation_needs_no_gpu():
    lib = L.load()
    p = ctypes.c_void_p(4096)
    ptrs = [p] * 10  # conv_state .. out
    ok_tail = (1, 1, 1, None)  # dtype, state_dtype, weight_dtype, stream
    assert lib.hawk_decode_block_step(None, 4096, *ptrs, 2, 2048, 128, 4, *ok_tail) == -1
    assert lib.hawk_decode_block_step(p, 4096, *ptrs, 2, 2048, 100, 4, *ok_tail) == -2   # R % block_width
    assert lib.hawk_decode_block_step(p, 2048, *ptrs, 2, 2048, 128, 4, *ok_tail) == -2   # row stride < 2R
    assert lib.hawk_decode_block_step(p, 4096, *ptrs, 2, 2048, 256, 4, *ok_tail) == -7   # block wider than 128
    assert lib.hawk_decode_block_step(p, 4096, *ptrs, 2, 2048, 128, 5, *ok_tail) == -7   # conv width
    assert lib.hawk_decode_block_step(p, 4096, *ptrs, 2, 2048, 128, 4, 1, 1, 9, None) == -3


def test_fused_scan_and_gate_projection_argument_validation_needs_no_gpu():
    lib = L.load()
    p = ctypes.c_void_p(4096)
    bf = L.HAWK_BF16
    # x gx ga lam | gate_bias | y, y strides | h out
    assert lib.hawk_scan_gelu_fwd(p, p, p, p, None, None, 8192, 128, p, p, 1, 8, 64, bf, None) == -1     # y missing
    assert lib.hawk_scan_gelu_fwd(p, p, p, p, None, p, 8192, 32, p, p, 1, 8, 64, bf, None) == -2         # row stride < D
    assert lib.hawk_scan_gelu_fwd(p, p, p, p, None, p, 8192, 132, p, p, 1, 8, 64, bf, None) == -4        # stride % 8
    assert lib.hawk_scan_gelu_fwd(p, p, p, p, None, ctypes.c_void_p(4100), 8192, 128, p, p, 1, 8, 64, bf, None) == -4
    assert lib.hawk_scan_gelu_fwd(p, p, p, p, None, p, 8192, 128, p, p, 1, 8, 96, bf, None) == -2        # D % 64
    # x gx ga lam gate_bias h | y, strides | dout dx dgx dga | dy, strides | dlam dgate_bias | workspace
    tail = (1, 8, 64, bf, None)
    assert lib.hawk_scan_gelu_bwd(p, p, p, p, None, p, p, 8192, 128, p, p, p, p, None, 8192, 128, p, None, p, 256, *tail) == -1
    assert lib.hawk_scan_gelu_bwd(p, p, p, p, None, p, p, 8192, 128, p, p, p, p, p, 8192, 128, p, None, p, 16, *tail) == -5
    assert lib.hawk_scan_gelu_bwd(p, p, p, p, p, p, p, 8192, 128, p, p, p, p, p, 8192, 128, p, p, p, 256, *tail) == -5  # 3 planes
    # gate projections: width a multiple of 128, block width dividing 128
    assert lib.hawk_gates_packed_bytes(2048, 128) == 16 * (256 * 128 + 128 * 384) * 2
    assert lib.hawk_gates_packed_bytes(2048, 96) == 0 and lib.hawk_gates_packed_bytes(192, 64) == 0
    assert lib.hawk_gates_pack_weights(p, p, 0, p, 2048, 48, None) == -2
    assert lib.hawk_gates_pack_weights(p, None, 0, p, 2048, 128, None) == -1
    assert lib.hawk_gates_pack_weights(p, p, 5, p, 2048, 128, None) == -3
    assert lib.hawk_gates_fwd(p, p, p, p, 4096, 2048, 128, None, None) == -1        # status word missing
    assert lib.hawk_gates_fwd(p, p, p, p, 4096, 1000, 8, p, None) == -2
    assert lib.hawk_gates_fwd(ctypes.c_void_p(4104), p, p, p, 4096, 2048, 128, p, None) == -4
    need = lib.hawk_gates_bwd_workspace_bytes(4096, 2048, 128)
    assert need >= 16 * 128 * 256 * 4
    assert lib.hawk_gates_bwd(p, p, p, p, p, p, p, p, need - 1, 4096, 2048, 128, p, None) == -5
    assert lib.hawk_debug_wait_timeout(p, 1024, 100000, p, None) == -5               # scratch too small
    assert lib.hawk_debug_wait_timeout(p, 1 << 20, 10, p, None) == -2                # budget out of range


def test_time_split_policy_and_validation_need_no_gpu():
    """hawk_scan_split_chunks is host arithmetic: its answers are ones the split entry points accept (a divisor of
    T, at most 64 pieces of at least 256 rows), it leaves launches with enough CTAs alone, and the entry points
    reject bad splits before touching the device."""
    lib = L.load()
    FWD, FWD_GELU, BWD = 0, 1, 2
    for which in (FWD, FWD_GELU, BWD):
        for (B, T, D) in [(1, 65536, 64), (1, 65536, 512), (2, 2048, 512), (1, 4096, 256), (3, 8192, 128), (1, 300, 64),
                          (1, 1021, 512), (8, 4096, 2048), (1, 65536, 4096), (64, 4096, 64)]:
            n = lib.hawk_scan_split_chunks(B, T, D, which)
            assert 1 <= n <= 64 and T % n == 0 and (n == 1 or T // n >= 256), (B, T, D, which, n)
        assert lib.hawk_scan_split_chunks(8, 4096, 2048, which) == 1
        assert lib.hawk_scan_split_chunks(1, 65536, 4096, which) == 1
        assert lib.hawk_scan_split_chunks(1, 65536, 512, which) > 1
        assert lib.hawk_scan_split_chunks(1, 1021, 512, which) == 1  # a prime number of rows cannot be cut evenly
    # 64 CTAs of 32 channels but 128 of 16: only the plain forward stays whole
    assert lib.hawk_scan_split_chunks(1, 65536, 2048, FWD) == 1 and lib.hawk_scan_split_chunks(1, 65536, 2048, BWD) > 1
    assert lib.hawk_scan_split_workspace_bytes(2, 8, 512) == 7 * 2 * 8 * 512 * 4
    assert lib.hawk_scan_split_workspace_bytes(0, 8, 512) == 0
    p = ctypes.c_void_p(4096)  # never dereferenced: validation fails first
    args = lambda nsub, wsb, T=1024: (p, p, p, p, None, None, None, 0, 0, p, None, nsub, p, wsb, 1, T, 64, 1, None)
    big = 1 << 30
    assert lib.hawk_scan_fwd_split(*args(3, big)) < 0               # 1024 rows do not split in three
    assert lib.hawk_scan_fwd_split(*args(65, big, T=65 * 64)) < 0   # more pieces than supported
    assert lib.hawk_scan_fwd_split(*args(4, 16)) < 0                # workspace too small
    assert lib.hawk_scan_fwd_split(p, p, p, p, None, None, p, 0, 0, p, None, 4, p, big, 1, 1024, 64, 1, None) < 0  # y without out


def test_reference_class_names_resolve_to_the_operators():
    """hawk/scan_fused.py:426-445 and hawk/fused_cross_entropy.py:11-79 expose their operators as
    `Class.apply`; the same spellings work here."""
    from hawk_b200 import ops
    assert ops.DiagonalRecurrence.apply is ops.fused_linear_scan
    assert ops.CrossEntropyLoopedFused.apply is ops.fused_cross_entropy
