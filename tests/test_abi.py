"""CPU: libixk.so loads without a GPU, exports every symbol include/ixk.h declares, and its
structs have the layout the Python mirror assumes.  No compute call is made."""
import ctypes
import os
import re
import subprocess
import sys
import tempfile

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "ixk.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ixk_[a-z0-9_]+)\s*\(", text)))


def test_header_functions_are_all_bound_and_exported(pkg):
    names = declared_functions()
    assert len(names) >= 10
    lib = ctypes.CDLL(pkg.library_path())
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in ixk.h but not exported"
    assert sorted(pkg.ABI_SYMBOLS) == names, "python mirror and header disagree"


def test_struct_layout_matches_c(pkg):
    """Compile a probe with the real header and compare sizeof/offsetof with ctypes."""
    src = r'''
#include <stdio.h>
#include <stddef.h>
#include "ixk.h"
int main(void) {
  printf("%zu %zu %zu\n", sizeof(ixk_matrix_layout), sizeof(ixk_gemm_desc), sizeof(ixk_fmha_desc));
  printf("%zu %zu %zu %zu\n", offsetof(ixk_gemm_desc, output), offsetof(ixk_gemm_desc, batch_size),
         offsetof(ixk_gemm_desc, beta), offsetof(ixk_gemm_desc, epilogue));
  printf("%zu %zu %zu\n", offsetof(ixk_fmha_desc, head_scale), offsetof(ixk_fmha_desc, q_strides),
         offsetof(ixk_fmha_desc, bias_strides));
  return 0;
}
'''
    with tempfile.TemporaryDirectory() as d:
        c = os.path.join(d, "probe.c")
        exe = os.path.join(d, "probe")
        open(c, "w").write(src)
        subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), c, "-o", exe],
                       check=True)
        out = subprocess.run([exe], check=True, capture_output=True, text=True).stdout.split()
    got = [int(x) for x in out]
    G, F = pkg._GemmDesc, pkg._FmhaDesc
    want = [ctypes.sizeof(pkg._MatrixLayout), ctypes.sizeof(G), ctypes.sizeof(F),
            G.output.offset, G.batch_size.offset, G.beta.offset, G.epilogue.offset,
            F.head_scale.offset, F.q_strides.offset, F.bias_strides.offset]
    assert got == want


def test_status_strings_and_version(pkg):
    lib = pkg.load_library()
    names = [lib.ixk_status_string(i).decode() for i in range(7)]
    assert names == ["OK", "INVALID_ARGUMENT", "UNIMPLEMENTED", "WORKSPACE_TOO_SMALL", "CUDA_ERROR", "NO_DEVICE",
                     "DEVICE_TIMEOUT"]
    assert lib.ixk_status_string(99).decode() == "UNKNOWN"
    assert re.fullmatch(r"\d+\.\d+\.\d+", pkg.version())


def test_workspace_queries_need_no_gpu(pkg):
    lib = pkg.load_library()
    d = pkg._FmhaDesc()
    d.dtype, d.num_batches, d.num_heads, d.head_size, d.num_queries, d.num_keys = 0, 64, 16, 256, 1, 4096
    # decode: ceil(16*148 / 1024) = 3 key splits, each a partial of (H + 2) floats per row
    assert lib.ixk_fmha_fwd_workspace_bytes(ctypes.byref(d)) == 3 * 64 * 16 * 1 * 258 * 4
    d.num_queries = 2048  # prefill keeps everything on chip
    assert lib.ixk_fmha_fwd_workspace_bytes(ctypes.byref(d)) == 0
    assert lib.ixk_gemm_workspace_bytes(None) == 0
    # backward: -lse*log2e, rowsum(dO*O) and the fp32 dQ accumulator over rows padded to 128 queries
    bd = pkg._FmhaBwdDesc()
    bd.fwd.dtype, bd.fwd.num_batches, bd.fwd.num_heads, bd.fwd.head_size = 0, 2, 3, 96
    bd.fwd.num_queries, bd.fwd.num_keys = 200, 77
    assert lib.ixk_fmha_bwd_workspace_bytes(ctypes.byref(bd)) == 2 * 3 * 256 * (128 + 2) * 4
    bd.fwd.head_size = 64
    assert lib.ixk_fmha_bwd_workspace_bytes(ctypes.byref(bd)) == 2 * 3 * 256 * (64 + 2) * 4
    # head sizes above 128: the two per-row arrays (rounded up to 256 bytes) + fp32 and 16-bit scores of
    # one group of heads, key pitch rounded up to 8 (here all 3 heads fit one group)
    bd.fwd.head_size = 256
    rows = 2 * 3 * 256 * 2 * 4
    assert rows % 256 == 0
    assert lib.ixk_fmha_bwd_workspace_bytes(ctypes.byref(bd)) == rows + 3 * 200 * 80 * 4 + 3 * 200 * 80 * 2
    assert lib.ixk_fmha_bwd_workspace_bytes(None) == 0


def test_argument_errors_come_back_as_codes_not_aborts(pkg):
    """Validation happens on the host before any launch (the reference CHECK-aborts instead,
    xetla_gpu_fused_mha_runner.cc:114-116)."""
    lib = pkg.load_library()
    assert lib.ixk_gemm(None, None, None, None, None, None, None, 0, None) == pkg.IXK_INVALID_ARGUMENT
    assert b"desc is NULL" in lib.ixk_last_error()
    g = pkg._GemmDesc()
    g.batch_size, g.alpha, g.epilogue = 1, 1.0, 6  # GELU_AUX
    assert lib.ixk_gemm(ctypes.byref(g), None, None, None, None, None, None, 0, None) == pkg.IXK_UNIMPLEMENTED
    assert b"ixk_gemm_aux" in lib.ixk_last_error()
    assert lib.ixk_gemm_aux(ctypes.byref(g), None, None, None, None, None, None, 0, None) == pkg.IXK_OK   # an empty problem
    g.epilogue = 42
    assert lib.ixk_gemm(ctypes.byref(g), None, None, None, None, None, None, 0, None) == pkg.IXK_INVALID_ARGUMENT
    g.epilogue = 0
    assert lib.ixk_gemm_aux(ctypes.byref(g), None, None, None, None, None, None, 0, None) == pkg.IXK_INVALID_ARGUMENT
    assert b"GELU_AUX" in lib.ixk_last_error()
    g.alpha = float("nan")
    assert lib.ixk_gemm(ctypes.byref(g), None, None, None, None, None, None, 0, None) == pkg.IXK_INVALID_ARGUMENT
    f = pkg._FmhaDesc()
    f.dtype, f.dropout_prob = 0, 0.1
    assert lib.ixk_fmha_fwd(ctypes.byref(f), None, None, None, None, None, None, None, 0, None) == pkg.IXK_UNIMPLEMENTED
    assert b"dropout" in lib.ixk_last_error()
    f.dropout_prob, f.head_size = 0.0, 512
    assert lib.ixk_fmha_fwd(ctypes.byref(f), None, None, None, None, None, None, None, 0, None) == pkg.IXK_UNIMPLEMENTED
    f.head_size, f.dtype = 64, 2  # F32
    assert lib.ixk_fmha_fwd(ctypes.byref(f), None, None, None, None, None, None, None, 0, None) == pkg.IXK_UNIMPLEMENTED
    assert lib.ixk_fmha_bwd(None, None, None, None, None, None, None, None, None, None, None, None, 0, None) \
        == pkg.IXK_INVALID_ARGUMENT
    bd = pkg._FmhaBwdDesc()
    bd.fwd.dtype, bd.fwd.dropout_prob = 0, 0.5
    assert lib.ixk_fmha_bwd(ctypes.byref(bd), None, None, None, None, None, None, None, None, None, None, None, 0,
                            None) == pkg.IXK_UNIMPLEMENTED
    assert lib.ixk_row_norm(2, 0, 4, 16, None, 16, None, 16, 1e-5, None) == pkg.IXK_UNIMPLEMENTED      # fp32
    assert lib.ixk_row_norm(0, 7, 4, 16, None, 16, None, 16, 1e-5, None) == pkg.IXK_INVALID_ARGUMENT  # kind
    assert lib.ixk_residual_add(0, 4, 12, None, None, None, None, None) == pkg.IXK_INVALID_ARGUMENT   # null, cols % 8
    assert lib.ixk_rotary_interleaved(0, None, 8, 3, 2, 32, 64, 64, None, None, None) == pkg.IXK_INVALID_ARGUMENT


def test_zero_strides_are_a_broadcast_only_where_that_is_a_read(pkg):
    """Stride 0 on a dimension with several entries: accepted for k / v over heads and batches
    (one K/V for all heads) and for the bias; refused for q, for the key rows and for everything
    that is written.  All on the host, before any pointer is looked at."""
    lib = pkg.load_library()

    def desc(**over):
        f = pkg._FmhaDesc()
        f.dtype, f.num_batches, f.num_heads, f.head_size, f.num_queries, f.num_keys = 0, 2, 4, 64, 128, 256
        f.head_scale = 0.125
        f.q_strides[:] = [4 * 128 * 64, 128 * 64, 64]
        f.o_strides[:] = [4 * 128 * 64, 128 * 64, 64]
        f.k_strides[:] = [4 * 256 * 64, 256 * 64, 64]
        f.v_strides[:] = [4 * 256 * 64, 256 * 64, 64]
        for name, val in over.items():
            getattr(f, name)[:] = val
        return f

    def fwd(f):
        return lib.ixk_fmha_fwd(ctypes.byref(f), None, None, None, None, None, None, None, 0, None)

    # with legal strides the call gets as far as the NULL pointers
    assert fwd(desc()) == pkg.IXK_INVALID_ARGUMENT and b"non-NULL" in lib.ixk_last_error()
    assert fwd(desc(k_strides=[0, 0, 64], v_strides=[256 * 64, 0, 64])) == pkg.IXK_INVALID_ARGUMENT
    assert b"non-NULL" in lib.ixk_last_error()                       # K/V shared between heads: accepted
    assert fwd(desc(q_strides=[4 * 128 * 64, 0, 64])) == pkg.IXK_UNIMPLEMENTED
    assert fwd(desc(k_strides=[4 * 256 * 64, 256 * 64, 0])) == pkg.IXK_UNIMPLEMENTED
    assert fwd(desc(o_strides=[4 * 128 * 64, 0, 64])) == pkg.IXK_INVALID_ARGUMENT
    assert b"overwrite" in lib.ixk_last_error()

    bd = pkg._FmhaBwdDesc()
    bd.fwd = desc(k_strides=[4 * 256 * 64, 0, 64])
    for name, t in (("do", 128), ("dq", 128), ("dk", 256), ("dv", 256)):
        getattr(bd, name + "_strides")[:] = [4 * t * 64, t * 64, 64]
    one = ctypes.c_void_p(256)   # never dereferenced: the stride check comes first
    args = [one] * 10
    assert lib.ixk_fmha_bwd(ctypes.byref(bd), *args, None, 0, None) == pkg.IXK_UNIMPLEMENTED   # dK would need a sum over heads
    bd.fwd = desc()
    bd.dk_strides[:] = [4 * 256 * 64, 0, 64]
    assert lib.ixk_fmha_bwd(ctypes.byref(bd), *args, None, 0, None) == pkg.IXK_INVALID_ARGUMENT


def test_python_descriptor_checks_that_shapes_agree(pkg):
    import torch
    q = torch.zeros(2, 4, 16, 64, dtype=torch.bfloat16)
    k1 = torch.zeros(2, 1, 32, 64, dtype=torch.bfloat16)
    with pytest.raises(pkg.IxkError, match="expand"):
        pkg._fmha_desc(q, k1, k1, None, q, 1.0, False, 0.0)           # one K head handed over as a smaller tensor
    ke = k1.expand(2, 4, 32, 64)
    d = pkg._fmha_desc(q, ke, ke, None, q, 1.0, False, 0.0)
    assert list(d.k_strides) == [32 * 64, 0, 64]
    with pytest.raises(pkg.IxkError):
        pkg._fmha_desc(q, ke, ke, None, q[:, :2], 1.0, False, 0.0)    # out with fewer heads
    with pytest.raises(pkg.IxkError, match="element type"):
        pkg._fmha_desc(q, ke.half(), ke, None, q, 1.0, False, 0.0)


def test_ffi_operand_selection(pkg):
    """Which buffer of "__cublas$lt$matmul" is which, as SyclLtMatmul unpacks them
    (sycl_custom_call.cc:167-205): lhs, rhs, [C iff beta != 0], [bias iff the epilogue adds one];
    D is result 1 when there is an auxiliary output (result 0), else result 0."""
    lib = pkg.load_library()
    ops = pkg._FfiOperands()
    E = {n: i for i, n in enumerate(pkg.EPILOGUES)}

    def pick(epi, beta, n_args, n_res):
        st = lib.ixk_ffi_select_operands(E[epi], beta, n_args, n_res, ctypes.byref(ops))
        return st, (ops.lhs_arg, ops.rhs_arg, ops.c_arg, ops.bias_arg, ops.d_result, ops.aux_result)

    assert pick("DEFAULT", 0.0, 2, 1) == (pkg.IXK_OK, (0, 1, -1, -1, 0, -1))
    assert pick("DEFAULT", 1.0, 3, 1) == (pkg.IXK_OK, (0, 1, 2, -1, 0, -1))
    assert pick("BIAS_GELU", 0.0, 3, 1) == (pkg.IXK_OK, (0, 1, -1, 2, 0, -1))
    assert pick("BIAS_RELU", 0.5, 4, 1) == (pkg.IXK_OK, (0, 1, 2, 3, 0, -1))
    assert pick("GELU_AUX", 0.0, 2, 2) == (pkg.IXK_OK, (0, 1, -1, -1, 1, 0))
    assert pick("BIAS_GELU_AUX", 1.0, 4, 2) == (pkg.IXK_OK, (0, 1, 2, 3, 1, 0))
    assert pick("BIAS", 1.0, 3, 1)[0] == pkg.IXK_INVALID_ARGUMENT          # the bias operand is missing
    assert pick("GELU_AUX", 0.0, 2, 1)[0] == pkg.IXK_INVALID_ARGUMENT      # no second result
    assert lib.ixk_ffi_select_operands(9, 0.0, 2, 1, ctypes.byref(ops)) == pkg.IXK_INVALID_ARGUMENT
    assert b"Unknown Epilogue" in lib.ixk_last_error()
    assert lib.ixk_ffi_select_operands(0, 0.0, 2, 1, None) == pkg.IXK_INVALID_ARGUMENT


def test_xla_ffi_shim_is_inert_without_xla_headers(pkg):
    """csrc/xla_ffi_shim.cc registers the XLA FFI handlers when XLA's headers are on the include
    path; without them (this repository's own build) it must compile to an empty object."""
    src = os.path.join(os.path.dirname(pkg.__file__), "csrc", "xla_ffi_shim.cc")
    with tempfile.TemporaryDirectory() as d:
        obj = os.path.join(d, "shim.o")
        subprocess.run(["g++", "-std=c++17", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), "-c", src, "-o", obj],
                       check=True)
        syms = subprocess.run(["nm", "--defined-only", obj], check=True, capture_output=True, text=True).stdout
    assert syms.strip() == ""


def test_all_reduce_slices_and_set_up_errors(pkg):
    """The two-shot all-reduce splits whole 16-byte vectors evenly and gives the remainder to the
    last rank (ccl_ops.cc:103-114); creating a communicator needs a device."""
    lib = pkg.load_library()
    b, e = ctypes.c_size_t(), ctypes.c_size_t()
    count = 8 * 1001 + 5                       # 1001 vectors of 8 bf16 and 5 loose elements
    covered = []
    for r in range(4):
        assert lib.ixk_all_reduce_slice(pkg.IXK_BF16, count, r, 4, ctypes.byref(b), ctypes.byref(e)) == pkg.IXK_OK
        covered.append((b.value, e.value))
    assert covered == [(0, 2000), (2000, 4000), (4000, 6000), (6000, count)]
    assert lib.ixk_all_reduce_slice(pkg.IXK_F32, 10, 0, 1, ctypes.byref(b), ctypes.byref(e)) == pkg.IXK_OK
    assert (b.value, e.value) == (0, 10)
    assert lib.ixk_all_reduce_slice(pkg.IXK_F32, 10, 3, 2, ctypes.byref(b), ctypes.byref(e)) == pkg.IXK_INVALID_ARGUMENT
    import torch
    if not torch.cuda.is_available():
        h = ctypes.c_void_p()
        assert lib.ixk_comm_create(0, 2, 1 << 20, ctypes.byref(h), None) == pkg.IXK_NO_DEVICE
        assert h.value is None
        assert lib.ixk_selftest_bounded_wait(1000, None, None) == pkg.IXK_NO_DEVICE
    assert lib.ixk_all_reduce(None, 0, 0, 0, None, 16, None) == pkg.IXK_INVALID_ARGUMENT
    assert lib.ixk_comm_destroy(None) == pkg.IXK_OK
    # the calls that came with the fused projection + exchange and the decode step: a NULL
    # communicator, a NULL descriptor and an unsupported type are answered with codes, GPU or not
    assert lib.ixk_comm_set_alternating(None, 1) == pkg.IXK_INVALID_ARGUMENT
    assert lib.ixk_all_reduce_scattered(None, pkg.IXK_BF16, 0, None, None, 0, 8, 8, None) == pkg.IXK_INVALID_ARGUMENT
    assert lib.ixk_reduce_scatter(None, pkg.IXK_BF16, 0, 0, None, 8, None) == pkg.IXK_INVALID_ARGUMENT
    assert lib.ixk_all_gather(None, pkg.IXK_BF16, None, 0, 8, None) == pkg.IXK_INVALID_ARGUMENT
    d = pkg._GemmDesc()
    assert lib.ixk_gemm_scatter(None, ctypes.byref(d), None, None, None, None, 0, None) == pkg.IXK_INVALID_ARGUMENT
    assert lib.ixk_gemm_geglu(None, None, None, None, 0, None, 0, None) == pkg.IXK_INVALID_ARGUMENT
    assert lib.ixk_gemm_geglu_workspace_bytes(None) == 0
    assert lib.ixk_kv_append(pkg.IXK_F32, 1, 1, 8, None, None, 8, 8, None, None, 8, 8, 8, 0, None) == pkg.IXK_UNIMPLEMENTED
    assert lib.ixk_kv_append(pkg.IXK_BF16, 1, 1, 8, None, None, 8, 8, None, None, 8, 8, 8, 0, None) == pkg.IXK_INVALID_ARGUMENT
    assert lib.ixk_row_norm_gain(pkg.IXK_BF16, pkg.NORM_RMS, 1, 8, None, 8, None, 1.0, None, 8, 1e-6, None) == pkg.IXK_INVALID_ARGUMENT
    assert lib.ixk_rotary_half(pkg.IXK_F32, None, 1, 1, 1, 16, 16, 16, None, None, None) == pkg.IXK_UNIMPLEMENTED


def test_missing_library_fails_loudly(pkg, monkeypatch):
    """No silent fallback: without libixk.so the package raises."""
    monkeypatch.setattr(pkg, "_LIB", None)
    monkeypatch.setattr(pkg, "library_path", lambda: "/nonexistent/libixk.so")
    with pytest.raises(pkg.IxkError, match="no CPU fallback"):
        pkg.load_library()


def test_cpu_tensors_are_rejected(pkg):
    import torch
    x = torch.zeros(8, 8, dtype=torch.bfloat16)
    with pytest.raises(pkg.IxkError, match="no CPU path"):
        pkg.gemm(x, x)
    q = torch.zeros(1, 1, 8, 64, dtype=torch.bfloat16)
    with pytest.raises(pkg.IxkError, match="no CPU path"):
        pkg.fmha_forward_kernel(None, q, q, q, None, None, 0.0, q.clone(), None, 1.0, False)


def test_oracle_is_not_imported_by_the_product(pkg):
    """The package must not reach into oracle/ (the oracle is test infrastructure)."""
    pkg_dir = os.path.dirname(pkg.__file__)
    for dirpath, _, files in os.walk(pkg_dir):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                assert "oracle" not in open(os.path.join(dirpath, f)).read().lower(), f
