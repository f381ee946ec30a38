"""Build the native libraries in-tree with nvcc / g++ (no JIT cache, no torch headers):

  xfastertransformer_b200/lib/libxft_b200_kernels.so   all sm_100a CUDA kernels, C ABI
  xfastertransformer_b200/lib/libxft_b200_core.so      C++ runtime (INI, loader, sequences, paged KV, samplers,
                                                        xft::Model C++ API)

  xfastertransformer_b200/lib/xft_runtime_selftest     (--selftest) native unit tests of the host-side runtime, built
                                                        with AddressSanitizer + UndefinedBehaviorSanitizer

Usage: python csrc/build.py [--force] [--verbose] [--selftest]
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
OUT = os.path.join(ROOT, "xfastertransformer_b200", "lib")
OBJ = os.path.join(ROOT, "build", "obj")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVFLAGS = ARCH + ["-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC", "--use_fast_math", "-Xptxas", "-v"]


def _newer(src, dst, deps=()):
    if not os.path.exists(dst):
        return True
    t = os.path.getmtime(dst)
    return any(os.path.getmtime(s) > t for s in (src,) + tuple(deps))


def _run(cmd, verbose):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        raise RuntimeError("build failed: " + cmd[-1])
    if verbose:
        sys.stderr.write(r.stderr)
    return r.stderr


def build(force=False, verbose=False):
    os.makedirs(OUT, exist_ok=True)
    os.makedirs(OBJ, exist_ok=True)
    kdir = os.path.join(HERE, "kernels")
    headers = tuple(os.path.join(kdir, f) for f in os.listdir(kdir) if f.endswith((".cuh", ".h")))
    cus = sorted(f for f in os.listdir(kdir) if f.endswith(".cu"))
    objs, jobs = [], []
    for f in cus:
        src, obj = os.path.join(kdir, f), os.path.join(OBJ, f[:-3] + ".o")
        objs.append(obj)
        if force or _newer(src, obj, headers):
            jobs.append([NVCC] + NVFLAGS + ["-c", src, "-o", obj])
    with ThreadPoolExecutor(max_workers=8) as ex:
        logs = list(ex.map(lambda c: _run(c, verbose), jobs))
    lib = os.path.join(OUT, "libxft_b200_kernels.so")
    if jobs or not os.path.exists(lib):
        _run([NVCC] + ARCH + ["-shared", "-o", lib] + objs + ["-lcudart"], verbose)
    # C++ runtime (links the kernel library; $ORIGIN rpath keeps the pair relocatable) and the example CLI
    cdir = os.path.join(HERE, "core")
    api = os.path.join(HERE, "api")
    ccs = sorted(f for f in os.listdir(cdir) if f.endswith(".cc")) if os.path.isdir(cdir) else []
    if ccs:
        core = os.path.join(OUT, "libxft_b200_core.so")
        srcs = [os.path.join(cdir, f) for f in ccs]
        hdrs = tuple(os.path.join(cdir, f) for f in os.listdir(cdir) if f.endswith(".h")) + \
            tuple(os.path.join(api, "xft", f) for f in os.listdir(os.path.join(api, "xft")))
        cxx = ["g++", "-O2", "-std=c++17", "-fPIC", "-I", api, "-I", cdir, "-I", "/usr/local/cuda/include"]
        link = ["-L", OUT, "-lxft_b200_kernels", "-L", "/usr/local/cuda/lib64", "-lcudart", "-Wl,-rpath,$ORIGIN",
                "-Wl,-rpath,/usr/local/cuda/lib64", "-ldl", "-lpthread"]
        if force or jobs or any(_newer(s, core, hdrs) for s in srcs):
            _run(cxx + ["-shared", "-o", core] + srcs + link, verbose)
        ex_src = os.path.join(ROOT, "examples", "cpp", "example.cpp")
        ex_bin = os.path.join(OUT, "xft_example")
        if os.path.exists(ex_src) and (force or _newer(ex_src, ex_bin, hdrs) or _newer(core, ex_bin)):
            _run(cxx + ["-o", ex_bin, ex_src, "-L", OUT, "-lxft_b200_core", "-lxft_b200_kernels", "-L",
                        "/usr/local/cuda/lib64", "-lcudart", "-Wl,-rpath,$ORIGIN", "-Wl,-rpath,/usr/local/cuda/lib64"], verbose)
        cb_src = os.path.join(ROOT, "examples", "cpp", "cb_check.cpp")
        cb_bin = os.path.join(OUT, "xft_cb_check")
        if os.path.exists(cb_src) and (force or _newer(cb_src, cb_bin, hdrs) or _newer(core, cb_bin)):
            _run(cxx + ["-o", cb_bin, cb_src, "-L", OUT, "-lxft_b200_core", "-lxft_b200_kernels", "-L",
                        "/usr/local/cuda/lib64", "-lcudart", "-Wl,-rpath,$ORIGIN", "-Wl,-rpath,/usr/local/cuda/lib64"], verbose)
        tp_src = os.path.join(ROOT, "examples", "cpp", "tp_check.cpp")
        tp_bin = os.path.join(OUT, "xft_tp_check")
        if os.path.exists(tp_src) and (force or _newer(tp_src, tp_bin, hdrs) or _newer(core, tp_bin)):
            _run(cxx + ["-o", tp_bin, tp_src, "-L", OUT, "-lxft_b200_core", "-lxft_b200_kernels", "-L",
                        "/usr/local/cuda/lib64", "-lcudart", "-lpthread", "-Wl,-rpath,$ORIGIN",
                        "-Wl,-rpath,/usr/local/cuda/lib64"], verbose)
        # torch custom-class binding (torch.classes.xfastertransformer.AutoModel) on top of the C++ runtime
        tb_src = os.path.join(api, "torch_binding.cc")
        tb_lib = os.path.join(OUT, "libxft_b200_torch.so")
        if os.path.exists(tb_src) and os.environ.get("XFT_BUILD_TORCH_BINDING", "1") != "0" and \
                (force or _newer(tb_src, tb_lib, hdrs) or _newer(core, tb_lib)):
            try:
                import torch
                from torch.utils import cpp_extension as ce
                inc = sum((["-isystem", d] for d in ce.include_paths()), [])
                tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
                abi = "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI)
                _run(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", abi, "-I", api, "-I", cdir] + inc +
                     ["-o", tb_lib, tb_src, "-L", OUT, "-lxft_b200_core", "-L", tlib, "-ltorch", "-ltorch_cpu", "-lc10",
                      "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + tlib], verbose)
            except ImportError:
                pass
    return lib, "".join(logs)


def build_selftest(verbose=False):
    """Native unit tests of the host-side runtime, compiled together with the runtime sources they cover under
    AddressSanitizer and UndefinedBehaviorSanitizer (the device-free part of the C++ core: no kernel library needed)."""
    os.makedirs(OUT, exist_ok=True)
    cdir = os.path.join(HERE, "core")
    src = os.path.join(HERE, "tests", "runtime_selftest.cc")
    out = os.path.join(OUT, "xft_runtime_selftest")
    srcs = [os.path.join(cdir, f) for f in ("runtime.cc", "ini.cc", "beam.cc", "env.cc", "arena.cc", "rope_tables.cc", "tokenizer.cc", "bpe_tokenizer.cc", "gptq.cc")]
    hdrs = tuple(os.path.join(cdir, f) for f in os.listdir(cdir) if f.endswith(".h"))
    if any(_newer(s, out, hdrs) for s in srcs + [src]):
        _run(["g++", "-O1", "-g", "-std=c++17", "-fsanitize=address,undefined", "-fno-sanitize-recover=undefined",
              "-fno-omit-frame-pointer", "-Wall", "-Wextra", "-Werror", "-I", cdir, "-I", "/usr/local/cuda/include",
              "-o", out, src] + srcs + ["-L", "/usr/local/cuda/lib64", "-lcudart", "-Wl,-rpath,/usr/local/cuda/lib64",
                                        "-lpthread"], verbose)
    return out


if __name__ == "__main__":
    if "--selftest" in sys.argv:
        print(build_selftest(verbose="--verbose" in sys.argv))
        sys.exit(0)
    lib, _ = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(lib)
