"""The C-ABI library builds for sm_100a, loads without a GPU and exports every declared symbol."""
import ctypes
import re
from pathlib import Path

from mflux_b200 import _lib

ROOT = Path(__file__).resolve().parent.parent


def _declared():
    names = set()
    for header in sorted((ROOT / "include").glob("*.h")):
        text = header.read_text()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names |= set(re.findall(r"\b(mfx_[a-z0-9_]+)\s*\(", text))
    return names


def test_library_exports_every_declared_symbol(lib_built):
    lib = _lib.load()
    declared = _declared()
    assert declared, "no declarations found in include/*.h"
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/ but not exported"
    assert declared == set(_lib.SIGNATURES), "ctypes signature table out of sync with include/*.h"


def test_version_and_status_strings(lib_built):
    lib = _lib.load()
    assert lib.mfx_version() == 100
    assert lib.mfx_status_str(0) == b"ok"
    for code in range(-9, 0):
        assert lib.mfx_status_str(code) != b"unknown status"


def test_argument_validation_needs_no_gpu(lib_built):
    """Host-side validation rejects bad calls before anything touches a device."""
    lib = _lib.load()
    assert lib.mfx_quantize_affine(None, 0, 4, 64, 4, 64, 0, None, None, None, None) == -7
    assert lib.mfx_quantize_affine(16, 0, 4, 64, 7, 64, 0, 16, 16, 16, None) == -3
    assert lib.mfx_quantize_affine(16, 0, 4, 64, 2, 64, 0, 16, 16, 16, None) == -3
    assert lib.mfx_quantize_affine(16, 0, 4, 96, 4, 64, 0, 16, 16, 16, None) == -1
    assert lib.mfx_quantize_affine(16, 0, 4, 64, 4, 32, 0, 16, 16, 16, None) == -3
    assert lib.mfx_quantize_affine(8, 0, 4, 64, 4, 64, 0, 16, 16, 16, None) == -2
    a = _lib.QLinearArgs()
    assert lib.mfx_qlinear_ex(a, None) == -7
    assert lib.mfx_qlinear_ex(None, None) == -7
    a.x = a.wq = a.scales = a.biases = a.y = a.workspace = 1024
    a.rows, a.batch, a.K, a.N, a.bits, a.group_size = 128, 1, 96, 64, 4, 64
    assert lib.mfx_qlinear_ex(a, None) == -1  # K % 64
    a.K = 128
    a.bits = 7
    assert lib.mfx_qlinear_ex(a, None) == -3
    a.bits = 4
    a.workspace_bytes = 16  # too small for the prepared form of the weight
    assert lib.mfx_qlinear_ex(a, None) == -1
    assert lib.mfx_qlinear_prepared_bytes(12288, 3072, 4, 64) == 12288 * 3072 // 2 + 12288 * 48 * 4
    assert lib.mfx_qlinear_prepared_bytes(12288, 3000, 4, 64) == 0
    # 3-bit codes are widened to 4 bits, 5- and 6-bit codes to 8 bits in the prepared form
    assert lib.mfx_qlinear_prepared_bytes(256, 128, 3, 64) == lib.mfx_qlinear_prepared_bytes(256, 128, 4, 64)
    assert lib.mfx_qlinear_prepared_bytes(256, 128, 5, 64) == lib.mfx_qlinear_prepared_bytes(256, 128, 8, 64)
    assert lib.mfx_qlinear_prepared_bytes(256, 128, 6, 64) == lib.mfx_qlinear_prepared_bytes(256, 128, 8, 64)
    assert lib.mfx_qlinear_prepared_bytes(256, 128, 7, 64) == 0
    assert lib.mfx_qlinear_prepared_bytes(10, 64, 4, 64) == 512 + 40  # 320 code bytes padded to 256s + pairs


def test_validation_of_the_later_entry_points(lib_built):
    """SwiGLU epilogue, post/pre-norm, gated residual, guidance combine and attention reject malformed calls on the
    host (status codes of include/mfx.h: -1 shape, -2 alignment, -4 dtype, -7 null, -9 too large)."""
    lib = _lib.load()
    a = _lib.QLinearArgs()
    a.x = a.wq = a.scales = a.biases = a.y = a.workspace = 1024
    a.rows, a.batch, a.K, a.N, a.bits, a.group_size = 128, 1, 128, 24, 4, 64
    a.workspace_bytes = 1 << 20
    a.x_row_stride, a.y_row_stride, a.y_dtype = 128, 24, _lib.BF16
    a.epilogue = _lib.EPI_SWIGLU
    assert lib.mfx_qlinear_ex(a, None) == -1          # N = 24 is not a multiple of 16
    a.epilogue = 7
    assert lib.mfx_qlinear_ex(a, None) == -1          # unknown epilogue
    a.epilogue = _lib.EPI_PEER_SCATTER
    assert lib.mfx_qlinear_ex(a, None) == -7          # tensor-parallel scatter without its descriptor
    sc = _lib.TpScatter()
    sc.world, sc.rank, sc.rows_per_rank, sc.D, sc.done_counter = 2, 0, 64, 24, 1024
    a.scatter = ctypes.pointer(sc)
    assert lib.mfx_qlinear_ex(a, None) == -7          # destination tables empty
    for r in range(2):
        sc.dst[r], sc.flags[r] = 1024, 1024
    sc.D = 32
    assert lib.mfx_qlinear_ex(a, None) == -1          # partial rows as wide as N
    sc.D, sc.rank = 24, 2
    assert lib.mfx_qlinear_ex(a, None) == -1          # rank outside the world
    sc.rank, sc.row_offset = 0, 64
    assert lib.mfx_qlinear_ex(a, None) == -1          # rows past the end of the joint sequence
    a.scatter = None
    f = _lib.TpFuseArgs()
    assert lib.mfx_tp_fuse(None, None) == -7
    assert lib.mfx_tp_fuse(f, None) == -1             # empty world
    f.world, f.rank, f.batch, f.rows_per_rank, f.seq_pad, f.seq, f.split, f.D = 2, 0, 1, 64, 128, 100, 20, 256
    assert lib.mfx_tp_fuse(f, None) == -7             # no residual rows
    f.x = f.done_counter = 1024
    f.mod_dtype = _lib.BF16
    f.seq = 129
    assert lib.mfx_tp_fuse(f, None) == -1             # more rows than the padded sequence
    f.seq, f.partials = 100, 1024
    assert lib.mfx_tp_fuse(f, None) == -7             # partial sums without gates
    assert lib.mfx_tp_wait(None, 2, 1, None, None) == -7
    assert lib.mfx_tp_wait(1024, 9, 1, None, None) == -1    # more ranks than MFX_TP_MAX_WORLD
    assert lib.mfx_tp_signal(None, 2, None) == -7
    ptrs = (ctypes.c_void_p * 2)(1024, None)
    assert lib.mfx_tp_signal(ptrs, 9, None) == -1           # more ranks than MFX_TP_MAX_WORLD
    assert lib.mfx_tp_signal(ptrs, 2, None) == -7           # a rank without a counter
    # low-rank term of the quantized matmul
    a.epilogue, a.N, a.y_row_stride = _lib.EPI_NONE, 64, 64
    a.lora_r = 8
    assert lib.mfx_qlinear_ex(a, None) == -7          # rank given without the two operands
    a.lora_t = a.lora_b = 1024
    a.lora_ld, a.lora_t_row_stride = 48, 48
    assert lib.mfx_qlinear_ex(a, None) == -1          # row length not a multiple of 64
    a.lora_ld, a.lora_t_row_stride = 64, 64
    a.lora_r = 65
    assert lib.mfx_qlinear_ex(a, None) == -1          # rank beyond the row length
    a.lora_r, a.lora_ld, a.lora_t_row_stride = 8, 2048, 2048
    assert lib.mfx_qlinear_ex(a, None) == -1          # more columns than the kernel takes
    a.lora_ld, a.lora_t_row_stride, a.lora_b = 64, 64, 1032
    assert lib.mfx_qlinear_ex(a, None) == -2          # operand not 16-byte aligned
    a.lora_b, a.lora_t_row_stride = 1024, 32
    assert lib.mfx_qlinear_ex(a, None) == -2          # rows of t shorter than the row length
    a.lora_r = -1
    assert lib.mfx_qlinear_ex(a, None) == -1
    p = _lib.PostPreNormArgs()
    assert lib.mfx_post_pre_norm(p, None) == -7
    assert lib.mfx_post_pre_norm(None, None) == -7
    p.y = p.weight = p.residual = 1024
    p.y_dtype, p.weight_dtype = _lib.BF16, _lib.BF16
    p.rows, p.batch, p.D = 4, 1, 100
    assert lib.mfx_post_pre_norm(p, None) == -1       # D % 8
    p.D = 8192
    assert lib.mfx_post_pre_norm(p, None) == -9       # wider than the kernel holds in registers
    p.D, p.y_row_stride, p.res_row_stride = 256, 256, 250
    assert lib.mfx_post_pre_norm(p, None) == -2       # residual rows not 16-byte aligned
    p.res_row_stride, p.y_dtype = 256, _lib.F16
    assert lib.mfx_post_pre_norm(p, None) == -4
    p.y_dtype, p.next_out = _lib.BF16, 2048
    assert lib.mfx_post_pre_norm(p, None) == -7       # second stage without its norm weight
    assert lib.mfx_gate_residual(1024, _lib.BF16, None, 0, 1024, _lib.BF16, 256, 1024, 1024, 250, 0, 1, 4, 256, None) == -2
    assert lib.mfx_gate_residual(1024, _lib.BF16, None, 0, 1024, _lib.BF16, 256, 1024, 1024, 128, 0, 1, 4, 256, None) == -1
    assert lib.mfx_gate_residual(None, _lib.BF16, None, 0, 1024, _lib.BF16, 256, 1024, 1024, 256, 0, 1, 4, 256, None) == -7
    assert lib.mfx_cfg_combine(1024, 1024, _lib.BF16, 3.0, 2, 1024, 4, 64, None) == -1   # unknown mode
    assert lib.mfx_cfg_combine(1024, 1024, _lib.BF16, 3.0, 0, 1024, 4, 2048, None) == -1  # more channels than a warp holds
    assert lib.mfx_fmha(1024, 1024, 1024, 384, 0, 0, 1, 1, 1.0, 1024, 128, 0, None) == -1
    assert lib.mfx_fmha(1024, 1024, 1028, 384, 0, 16, 1, 1, 1.0, 1024, 128, 0, None) == -2
    assert lib.mfx_qknorm_rope_gqa(1024, 1024, 0, 4, 1, 4, 8, 0, 0, 1024, 1024, 1024, 1024, _lib.F32, 1024, 1e-5, None) == -1
    assert lib.mfx_qknorm_rope_gqa(1024, 512, 0, 4, 1, 4, 2, 0, 0, 1024, 1024, 1024, 1024, _lib.F32, 1024, 1e-5, None) == -1
    assert lib.mfx_act_mul(1024, 256, 0, 1024, 256, 0, 4, 1, 100, 0, None) == -1     # D not a multiple of 8
    assert lib.mfx_act_mul(1024, 250, 0, 1024, 256, 0, 4, 1, 128, 0, None) == -2
    assert lib.mfx_act_mul(None, 256, 0, 1024, 256, 0, 4, 1, 128, 0, None) == -7
    assert lib.mfx_act_mul(1024, 256, 0, 1024, 256, 0, 4, 1, 128, 2, None) == -1    # unknown activation
    assert lib.mfx_qknorm_rope_gqa(1024, 1024, 0, 4, 1, 4, 2, 2, 0, 1024, 1024, 1024, 1024, _lib.F32, 1024, 1e-5, None) == -1
    assert lib.mfx_fmha_ex(None, None) == -7
    f = _lib.FmhaArgs()
    f.q = f.k = f.v = f.out = 1024
    f.q_row_stride = f.kv_row_stride = f.out_row_stride = 512
    f.seq_q, f.seq_kv, f.batch, f.heads, f.kv_heads, f.scale = 64, 96, 1, 4, 3, 1.0
    assert lib.mfx_fmha_ex(f, None) == -1             # 4 query heads over 3 key/value heads
    f.kv_heads = 2
    f.seq_kv = 0
    assert lib.mfx_fmha_ex(f, None) == -1             # no keys
    f.seq_kv, f.kv_row_stride = 96, 260
    assert lib.mfx_fmha_ex(f, None) == -2             # key rows not 16-byte aligned
    assert lib.mfx_vec_sum_act(1024, None, None, _lib.BF16, 3, 1024, _lib.BF16, 8, None) == -1
