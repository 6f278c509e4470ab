"""Builds functs_b200/_C*.so: the TorchScript pass module + immut:: operator registrations (g++, links the C-ABI
library next to it).  Run after functs_b200/build.py."""
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(os.path.dirname(HERE))
OUT = os.path.join(PKG, "_C" + sysconfig.get_config_var("EXT_SUFFIX"))
SOURCES = ["immut_ops.cpp", "tensorssa.cpp", "fusion.cpp", "regions.cpp", "generic_group.cpp", "shape_infer.cpp", "module.cpp"]


def stale() -> bool:
    if not os.path.exists(OUT):
        return True
    built = os.path.getmtime(OUT)
    deps = [os.path.join(HERE, f) for f in os.listdir(HERE) if f.endswith((".cpp", ".h", ".inc"))]
    deps.append(os.path.join(PKG, "..", "include", "functs_b200.h"))
    return any(os.path.getmtime(d) > built for d in deps)


def build(force: bool = False) -> str:
    if not force and not stale():
        return OUT
    import torch
    from torch.utils import cpp_extension as ce
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    objs = []
    flags = ["-O2", "-std=c++17", "-fPIC", "-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H",
             f"-D_GLIBCXX_USE_CXX11_ABI={int(torch.compiled_with_cxx11_abi())}", "-Wno-deprecated-declarations"]
    incs = [f"-I{p}" for p in ce.include_paths()] + [f"-I{sysconfig.get_paths()['include']}", "-I/usr/local/cuda/include"]
    procs = []
    for src in SOURCES:
        obj = os.path.join(HERE, src.replace(".cpp", ".o"))
        objs.append(obj)
        procs.append((src, subprocess.Popen(["g++", "-c", os.path.join(HERE, src), "-o", obj] + flags + incs,
                                            stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            raise RuntimeError(f"g++ failed on {src}:\n{out}")
    link = ["g++", "-shared", "-o", OUT] + objs + [f"-L{tlib}", "-ltorch", "-ltorch_cpu", "-lc10", "-lc10_cuda",
                                                  "-ltorch_python", f"-L{PKG}", "-lfuncts_b200",
                                                  f"-Wl,-rpath,{tlib}", "-Wl,-rpath,$ORIGIN"]
    res = subprocess.run(link, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("link failed:\n" + res.stdout + res.stderr)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
