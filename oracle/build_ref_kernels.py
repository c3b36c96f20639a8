"""Builds oracle/_ref/libref_kernels.so: the reference's OWN CUDA kernels for LayerNorm, RMSNorm, RoPE, Softmax,
IndexSelect and the triangular masks, fp32 and fp16, compiled for sm_100a.

The reference keeps these kernels as CUDA C text inside two C# verbatim strings (`Code` and `CodeHalf` of
TensorSharp.CUDA/DeviceCode/AdvFuncKernels.cs, compiled at run time with NVRTC).  This recipe reads that file where it
lies in the reference checkout, undoes the C# quoting (`""` -> `"`), writes the text to oracle/_ref/ (git-ignored:
reference source never enters the repository) and compiles it together with oracle/ref_launch.cu, a launcher that
starts each kernel with the launch shape the reference's host code uses.  The result is test infrastructure: the GPU
tests use it to pin the CPU oracle and the library's kernels against outputs of the reference's kernels themselves.

    python oracle/build_ref_kernels.py [/path/to/reference]
"""
import os
import re
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
LIB = os.path.join(OUT, "libref_kernels.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
SOURCE = "TensorSharp.CUDA/DeviceCode/AdvFuncKernels.cs"


def extract(cs_text, name):
    """The body of `private static readonly string <name> = @"...";` with the verbatim-string quoting undone."""
    m = re.search(r'private static readonly string %s = @"' % re.escape(name), cs_text)
    if not m:
        raise RuntimeError("string %s not found in %s" % (name, SOURCE))
    i = m.end()
    out = []
    while True:
        j = cs_text.index('"', i)
        out.append(cs_text[i:j])
        if cs_text[j:j + 2] == '""':
            out.append('"')
            i = j + 2
        else:
            break
    return "".join(out)


def build(reference_root="/root/reference", force=False):
    src = os.path.join(reference_root, SOURCE)
    if not os.path.exists(src):
        return LIB if os.path.exists(LIB) else None       # no reference checkout here: use what was built earlier
    os.makedirs(OUT, exist_ok=True)
    launcher = os.path.join(HERE, "ref_launch.cu")
    if (not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= max(os.path.getmtime(src), os.path.getmtime(launcher),
                                                                           os.path.getmtime(__file__))):
        return LIB
    with open(src, encoding="utf-8-sig") as fh:
        text = fh.read()
    # the order in which the reference concatenates the strings for an fp16 context (AdvFuncKernels.cs:2481-2489)
    code = extract(text, "Code") + "\n" + extract(text, "CodeHalf")
    with open(os.path.join(OUT, "adv_func_kernels_extracted.cu"), "w") as fh:
        fh.write(code)
    cmd = [NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-shared", "-Xcompiler", "-fPIC",
           "-I", OUT, launcher, "-o", LIB, "-cudart", "static"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed on the extracted reference kernels:\n%s\n%s" % (r.stdout, r.stderr[-4000:]))
    return LIB


if __name__ == "__main__":
    print(build(*(sys.argv[1:2]), force=True))
