"""The drop-in boundary, checked without a GPU: the library builds, loads, exports
every symbol that include/sideaware.h declares (and that the reference exports,
sideaware.cu:1278-1524), fails loudly instead of falling back when there is no
device, and compiles functor headers for sm_100a through NVRTC."""
import os
import re

import pytest

import l2_torch_alloc_b200 as pkg
from l2_torch_alloc_b200 import _binding, build, functors

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# the 26 entry points of the reference's extern "C" block
REFERENCE_SYMBOLS = """
sideaware_malloc_async sideaware_free_async sideaware_malloc sideaware_free sideaware_release_unused
sideaware_malloc_auto sideaware_free_auto sideaware_elementwise sideaware_one_to_one sideaware_memcpy
sideaware_create_kernel_advanced sideaware_create_kernel sideaware_compression sideaware_alloc_threshold
sideaware_prealloc_config sideaware_free_mapped_thresholds sideaware_write_sass sideaware_fill_side_index
sideaware_gpu_side_index sideaware_cpu_side_index sideaware_sm_side_summary sideaware_num_sms
sideaware_num_sm_side0 sideaware_num_sm_side1 sideaware_min_sm_per_side sideaware_hash_mask
""".split()


@pytest.fixture(scope="module")
def sa():
    build.build()
    return pkg.SideAware()


def header_symbols():
    text = open(os.path.join(ROOT, "include", "sideaware.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(sideaware_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_every_reference_symbol():
    declared = set(header_symbols())
    assert len(REFERENCE_SYMBOLS) == 26
    assert set(REFERENCE_SYMBOLS) <= declared


def test_library_exports_every_declared_symbol(sa):
    for name in header_symbols():
        assert hasattr(sa.lib, name), f"{name} declared in sideaware.h but not exported"
    assert set(header_symbols()) == set(_binding.SIGNATURES), "ctypes table and header disagree"


def test_no_device_is_a_loud_error_not_a_fallback(sa):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    before = sa.error_count()
    with pytest.raises(RuntimeError, match="no CUDA device|cannot"):
        sa.summary()
    assert sa.error_count() > before
    with pytest.raises(MemoryError):
        sa.malloc(16 << 20)


def test_missing_library_is_a_loud_error(tmp_path):
    with pytest.raises(FileNotFoundError, match="build it"):
        pkg.SideAware(str(tmp_path / "sideaware.so"))


def test_create_kernel_registry_needs_no_gpu(sa):
    assert sa.create_kernel(b"") == 0  # id 0 is memcpy (sideaware.cu:1422-1424)
    a = sa.create_kernel(functors.MEMCPY)
    b = sa.create_kernel(functors.silu_mul_bf16())
    assert a >= 1 and b >= 1 and a != b
    assert sa.create_kernel(functors.MEMCPY) == a  # same text, same id (sideaware.cu:1434-1438)


# the functor of the reference's own test (test.py:191-216), restated: mixed element sizes,
# two outputs, reverse order, all inputs streamed
MIXED_HEADER = b"""
#include <cuda_fp16.h>
#include <cuda_bf16.h>
typedef float o0;
typedef half o1;
typedef __nv_bfloat16 i0;
typedef float i1;
struct unused {};
typedef unused o2, o3, i2, i3;
__device__ void elementwise_op(size_t element_idx, int sideband, o0 &out0, o1 &out1, o2 &out2, o3 &out3,
                               const i0 &in0, const i1 &in1, const i2 &in2, const i3 &in3) {
    out0 = (o0)((float)in0 + (float)in1);
    out1 = (o1)((float)in1 * 10.0f);
}
constexpr bool reverse_order = true;
constexpr bool input_evict[4] = {1,1,1,1};
"""


@pytest.mark.parametrize("wide", [False, True])
def test_functor_headers_compile_for_sm100a(sa, wide):
    headers = {
        "memcpy": functors.MEMCPY,
        "mixed": MIXED_HEADER,
        "silu_mul": functors.silu_mul_bf16(),
        "rope_f32_mha": functors.rope_forward(1024, 32, 32, 128, False),
        "rope_bf16_gqa": functors.rope_forward(8192, 32, 8, 128, True),
        "knobs": functors.MEMCPY + "\n#define DISCARD_INPUTS\nconstexpr bool input_discard[4] = {1,0,0,0};\n"
                 "#define FORCE_WRONG_SIDE true\n#define LAUNCH_BOUNDS __launch_bounds__(512, 1)\n#define UNROLLED 8\n",
    }
    for name, h in headers.items():
        log = sa.compile_check(h, wide)
        assert log == "", f"{name}: {log[:2000]}"


def test_bad_header_reports_the_compiler_log(sa):
    log = sa.compile_check(b"typedef int o0; this is not CUDA;")
    assert "error" in log.lower()


def test_cpp_header_instantiates_and_links(tmp_path):
    """include/sideaware.hpp: the templated conveniences compile and link against the library
    (the reference's kernel wrappers, sideaware.cu:1549-1570, cannot be instantiated)."""
    import subprocess
    src = tmp_path / "use.cpp"
    src.write_text("""
#include "sideaware.hpp"
int main(int argc, char**) {
    float* p = nullptr;
    if (argc > 100) {
        sideaware::malloc(&p, 1024);
        sideaware::malloc_async(&p, 1024);
        sideaware::memcpy(p, (const float*)p, 256);
        sideaware::one_to_one(0, p, (const float*)p, 1024);
        sideaware::elementwise(0, 1024, p, nullptr, nullptr, nullptr, p);
        sideaware::free_async(p);
        sideaware::free(p);
    }
    return sideaware_create_kernel("") == 0 ? 0 : 1;
}
""")
    libdir = os.path.join(ROOT, "l2_torch_alloc_b200")
    exe = tmp_path / "use"
    subprocess.check_call(["g++", "-std=c++17", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), str(src),
                           "-L", libdir, "-l:sideaware.so", f"-Wl,-rpath,{libdir}", "-o", str(exe)])
    assert subprocess.run([str(exe)]).returncode == 0


# ---------------------------------------------------------------------------
# the allocator-only library (counterpart of the reference's sideaware_alloc.cu)
# ---------------------------------------------------------------------------
ALLOC_ONLY_REFERENCE_SYMBOLS = """
sideaware_malloc_async sideaware_free_async sideaware_malloc sideaware_free sideaware_release_unused
sideaware_compression sideaware_prealloc_config sideaware_free_mapped_thresholds sideaware_fill_side_index
sideaware_gpu_side_index sideaware_cpu_side_index sideaware_sm_side_summary sideaware_num_sms
sideaware_num_sm_side0 sideaware_num_sm_side1 sideaware_min_sm_per_side sideaware_hash_mask
""".split()  # extern "C" block of sideaware_alloc.cu:692-762


def alloc_header_symbols():
    text = open(os.path.join(ROOT, "include", "sideaware_alloc.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(sideaware_[a-z0-9_]+)\s*\(", text)))


def test_allocator_only_library_exports_what_its_header_declares():
    import ctypes
    import subprocess
    path = build.build(alloc_only=True)
    lib = ctypes.CDLL(path)  # loads without a GPU and without NVRTC
    declared = alloc_header_symbols()
    assert set(ALLOC_ONLY_REFERENCE_SYMBOLS) <= set(declared)
    assert set(declared) <= set(header_symbols()), "the two headers must declare the same functions under the same names"
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in sideaware_alloc.h but not exported by sideaware_alloc.so"
    exported = subprocess.run(["nm", "-D", "--defined-only", path], capture_output=True, text=True, check=True).stdout
    exported = sorted(set(re.findall(r" T (sideaware_[a-z0-9_]+)", exported)))
    assert exported == declared, "exports and header disagree"
    for absent in ("sideaware_elementwise", "sideaware_memcpy", "sideaware_create_kernel", "sideaware_rope_forward"):
        assert absent not in exported
    lib.sideaware_last_error.restype = ctypes.c_char_p
    lib.sideaware_malloc_auto.restype = ctypes.c_void_p
    lib.sideaware_malloc_auto.argtypes = [ctypes.c_size_t, ctypes.c_int, ctypes.c_void_p]
    import torch
    if not torch.cuda.is_available():
        assert not lib.sideaware_malloc_auto(16 << 20, 0, None)  # loud failure, no fallback
        assert b"CUDA" in lib.sideaware_last_error() or b"device" in lib.sideaware_last_error()


def test_headers_compile_as_c_and_together_as_cxx(tmp_path):
    import subprocess
    inc = os.path.join(ROOT, "include")
    c_file = tmp_path / "only_alloc.c"
    c_file.write_text('#include "sideaware_alloc.h"\nint main(void) { sideaware_stats_t s; (void)s; return sideaware_num_sms() < 0; }\n')
    subprocess.run(["gcc", "-std=c11", "-Wall", "-Werror", "-I", inc, "-c", str(c_file), "-o", str(tmp_path / "a.o")], check=True)
    c_full = tmp_path / "full.c"
    c_full.write_text('#include "sideaware.h"\nint main(void) { return sideaware_num_sms() < 0; }\n')
    subprocess.run(["gcc", "-std=c11", "-Wall", "-Werror", "-I", inc, "-c", str(c_full), "-o", str(tmp_path / "c.o")], check=True)
    cxx_file = tmp_path / "both.cpp"
    cxx_file.write_text('#include "sideaware.h"\n#include "sideaware_alloc.h"\n#include "sideaware.h"\nint main() { sideaware_stats_t s; (void)s; return 0; }\n')
    subprocess.run(["g++", "-std=c++17", "-Wall", "-Werror", "-I", inc, "-c", str(cxx_file), "-o", str(tmp_path / "b.o")], check=True)


def test_compile_check_warns_about_group_wide_constructs():
    """Blocks are one-dimensional and a warp owns a chunk: a header that indexes by threadIdx.y or synchronises a
    256-thread group (uses the reference's launch shape allowed, sideaware.cu:83, :1407) is reported when it is checked."""
    import ctypes
    import l2_torch_alloc_b200 as pkg
    from l2_torch_alloc_b200 import functors
    sa = pkg.SideAware()
    buf = ctypes.create_string_buffer(1 << 14)
    assert sa.lib.sideaware_compile_check(functors.MEMCPY.encode(), 0, buf, len(buf)) == 0 and buf.value == b""
    grouped = functors.MEMCPY.replace("out0 = in0;", "out0 = in0 + (int)threadIdx.y; __syncthreads();")
    assert sa.lib.sideaware_compile_check(grouped.encode(), 0, buf, len(buf)) == 0  # it still compiles
    text = buf.value.decode()
    assert "warning" in text and "threadIdx.y" in text and "__syncthreads" in text
    with pytest.warns(UserWarning, match="one-dimensional"):
        assert sa.compile_check(grouped) == ""
