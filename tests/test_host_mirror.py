"""The C++17 mirror of the reference operator API (qwen3x-orin_b200/host): builds, keeps the
reference's argument limits and dispatch / binding rules (all host-side, no GPU needed), and -- where a
reference checkout exists -- defines exactly the symbols the reference's own headers declare."""
import importlib
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "qwen3x-orin_b200")
HOST = os.path.join(PKG, "host")
REFERENCE = os.environ.get("Q3X_REFERENCE_DIR") or os.path.abspath(os.path.join(ROOT, "..", "reference"))


@pytest.fixture(scope="module")
def host_lib():
    build = importlib.import_module("qwen3x-orin_b200.build")
    build.build_all()
    assert os.path.exists(build.HOST_LIB)
    return build.HOST_LIB


def compile_and_run(tmp_path, source, includes):
    exe = str(tmp_path / "t")
    cmd = ["g++", "-std=c++17", "-O1", "-Wall", "-Wextra", "-Werror", source, "-o", exe]
    for inc in includes:
        cmd += ["-I", inc]
    cmd += ["-L", PKG, "-lq3x_b200_host", "-lq3x_b200", f"-Wl,-rpath,{PKG}", "-Wl,--no-undefined"]
    subprocess.run(cmd, check=True, capture_output=True, text=True)
    return subprocess.run([exe], capture_output=True, text=True)


def test_mirror_argument_limits_dispatch_and_bindings(host_lib, tmp_path):
    out = compile_and_run(tmp_path, os.path.join(ROOT, "tests", "host", "host_mirror_test.cpp"),
                          [HOST, os.path.join(ROOT, "include")])
    assert out.returncode == 0, out.stdout + out.stderr
    assert "host mirror tests passed" in out.stdout


HAVE_REFERENCE = os.path.isdir(os.path.join(REFERENCE, "include", "q3x"))


@pytest.mark.skipif(not HAVE_REFERENCE, reason="no reference checkout")
def test_mirror_defines_the_reference_symbols(host_lib, tmp_path):
    """Every launcher address is taken through the REFERENCE's declarations and must resolve at link time; the
    projection composites come from q3x_b200_dispatch.cpp compiled against the reference's own model_weights.h."""
    ref_inc = os.path.join(REFERENCE, "include")
    obj = str(tmp_path / "dispatch_ref.o")
    subprocess.run(["g++", "-std=c++17", "-O1", "-Wall", "-Wextra", "-Werror", "-DQ3X_B200_USE_REFERENCE_HEADERS", "-I", ref_inc,
                    "-I", HOST, "-I", os.path.join(ROOT, "include"), "-c", os.path.join(HOST, "q3x_b200_dispatch.cpp"),
                    "-o", obj], check=True, capture_output=True, text=True)
    exe = str(tmp_path / "t")
    cmd = ["g++", "-std=c++17", "-O1", "-Wall", "-Wextra", "-Werror", os.path.join(ROOT, "tests", "host", "reference_symbols.cpp"),
           obj, "-o", exe, "-I", ref_inc, "-I", os.path.join(REFERENCE, "src", "kernels", "reference"),
           "-L", PKG, "-lq3x_b200_host", "-lq3x_b200", f"-Wl,-rpath,{PKG}", "-Wl,--no-undefined"]
    subprocess.run(cmd, check=True, capture_output=True, text=True)
    out = subprocess.run([exe], capture_output=True, text=True)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "71 reference launcher symbols resolved" in out.stdout


@pytest.mark.skipif(not HAVE_REFERENCE, reason="no reference checkout")
def test_binding_types_have_the_reference_layout(tmp_path):
    """Enumerator values, struct sizes, alignments and field offsets of the prefill operator binding types: the
    same 110 numbers from the mirror header and from the reference's own headers."""
    src = os.path.join(ROOT, "tests", "host", "bindings_layout_dump.cpp")
    outputs = []
    for name, flags in (("mirror", ["-I", HOST]), ("reference", ["-DUSE_REFERENCE_HEADERS", "-I", os.path.join(REFERENCE, "include")])):
        exe = str(tmp_path / name)
        subprocess.run(["g++", "-std=c++17", "-Wno-invalid-offsetof", *flags, src, "-o", exe], check=True, capture_output=True,
                       text=True)
        outputs.append(subprocess.run([exe], capture_output=True, text=True, check=True).stdout)
    assert outputs[0] == outputs[1]
    assert len(outputs[0].splitlines()) >= 100


@pytest.mark.gpu
def test_mirror_launchers_on_the_gpu_match_the_c_abi(host_lib, tmp_path):
    """One launcher of every family called through libq3x_b200_host.so with real device buffers; the
    bytes must equal those of the same call made on the C ABI (a wrong argument order in the forwarding
    code cannot pass)."""
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    exe = str(tmp_path / "host_gpu_test")
    cmd = ["g++", "-std=c++17", "-O1", "-Wall", "-Wextra", os.path.join(ROOT, "tests", "host", "host_gpu_test.cpp"),
           "-o", exe, "-I", HOST, "-I", os.path.join(ROOT, "include"), "-I", os.path.join(cuda_home, "include"),
           "-L", PKG, "-lq3x_b200_host", "-lq3x_b200", f"-Wl,-rpath,{PKG}",
           "-L", os.path.join(cuda_home, "lib64"), "-lcudart", f"-Wl,-rpath,{os.path.join(cuda_home, 'lib64')}"]
    subprocess.run(cmd, check=True, capture_output=True, text=True)
    out = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    if out.returncode == 77:
        pytest.skip(out.stdout.strip())
    assert out.returncode == 0, out.stdout[-4000:] + out.stderr[-2000:]
    assert "host mirror GPU tests passed" in out.stdout
