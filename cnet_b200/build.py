"""Builds libcnet_b200.so in-tree: the sm_100a kernels + C ABI (csrc/) and the C++ host
facade (host/).  ``python -m cnet_b200.build`` or ``build(force=True)``."""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "libcnet_b200.so")
CSRC = ["context.cu", "elementwise.cu", "rowreduce.cu", "embed.cu", "cgemm_simt.cu", "cgemm_tc.cu", "linear.cu", "fft.cu", "fft_pipe.cu", "cgemv_skinny.cu", "dp_allreduce.cu"]
HOST = ["cnet.cpp", "capi.cpp", "dp_nccl.cpp", "model_saver.cpp", "data_reader.cpp"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O3", "-lineinfo",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall"]


def _sources():
    src = [os.path.join(HERE, "csrc", f) for f in CSRC] + [os.path.join(HERE, "host", f) for f in HOST]
    deps = src + [os.path.join(HERE, "csrc", "common.cuh"), os.path.join(HERE, "host", "cnet.h"), os.path.join(HERE, "host", "dp_nccl.h"), os.path.join(HERE, "host", "data_reader.h"),
                  os.path.join(HERE, "..", "include", "cnet_b200.h"),
                  os.path.join(HERE, "..", "include", "cnet_b200_host.h")]
    return src, deps


def up_to_date():
    if not os.path.exists(LIB):
        return False
    t = os.path.getmtime(LIB)
    return all(os.path.getmtime(d) <= t for d in _sources()[1] if os.path.exists(d))


def build(force=False, verbose=False):
    if not force and up_to_date():
        return LIB
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    obj_dir = os.path.join(HERE, "build")
    os.makedirs(obj_dir, exist_ok=True)
    src, _ = _sources()
    objs, procs = [], []
    env = dict(os.environ)
    env.pop("CXX", None)
    env.pop("CC", None)
    for s in src:
        o = os.path.join(obj_dir, os.path.basename(s) + ".o")
        objs.append(o)
        cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", s, "-o", o]
        if s.endswith(".cpp"):
            cmd = [nvcc, "-std=c++17", "-O2", "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall", "-c", s, "-o", o]
        procs.append((s, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, env=env)))
    for s, p in procs:
        out = p.communicate()[0].decode()
        if p.returncode != 0:
            raise RuntimeError("nvcc failed on %s:\n%s" % (s, out))
        if verbose and out.strip():
            print(out)
    cmd = [nvcc, "-shared", "-o", LIB] + objs + ["-lcudart", "-ldl"]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, env=env)
    if r.returncode != 0:
        raise RuntimeError("link failed:\n" + r.stdout.decode())
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
