"""Builds the native pieces in-tree:

  graphtok_b200/lib/libgtok.so      CUDA kernels + engine + C ABI, sm_100a only
  graphtok_b200/datagen/datagen     synthetic text / vocabulary generator (host only)
  graphtok_b200/cli/gpu_bpe_tokenize   command-line tool over libgtok.so

nvcc cross-compiles without a GPU.  Run as `python -m graphtok_b200.build`.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
LIB = os.path.join(LIB_DIR, "libgtok.so")
DATAGEN = os.path.join(HERE, "datagen", "datagen")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O3", "-lineinfo",
    "-Xcompiler", "-fPIC", "--shared",
    "-Xlinker", "--version-script=" + os.path.join(CSRC, "gtok.map"),
]
SOURCES = ["encode_kernels.cu", "tiny_kernel.cu", "engine.cu", "gtok_abi.cc", "vocab_host.cc", "tables_build.cc", "nfc_host.cc"]


def _newer(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def source_hash():
    """Short hash of the native sources (csrc/ and the C ABI header): identifies the build a
    measurement or a profile summary was taken from."""
    import hashlib
    h = hashlib.sha256()
    for name in sorted(os.listdir(CSRC)):
        if name.endswith((".h", ".cu", ".cc", ".map")):
            with open(os.path.join(CSRC, name), "rb") as f:
                h.update(name.encode() + b"\0" + f.read())
    with open(os.path.join(HERE, "..", "include", "gtok.h"), "rb") as f:
        h.update(f.read())
    return h.hexdigest()[:16]


def _nvcc():
    return shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"


def build_lib(force=False, verbose=False):
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(HERE, "..", "include", "gtok.h")]
    if not force and not _newer(LIB, deps):
        return LIB
    os.makedirs(LIB_DIR, exist_ok=True)
    cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-o", LIB] + [os.path.join(CSRC, s) for s in SOURCES]
    subprocess.run(cmd, check=True)
    return LIB


def build_datagen(force=False):
    src = [os.path.join(HERE, "datagen", f) for f in ("datagen.cc", "seqsplit.h")] + [os.path.join(CSRC, f) for f in ("unicode_class_table.h", "unicode_wide_table.h")]
    if not force and not _newer(DATAGEN, src):
        return DATAGEN
    subprocess.run(["g++", "-std=c++17", "-O2", "-o", DATAGEN, src[0]], check=True)
    return DATAGEN


CLI = os.path.join(HERE, "cli", "gpu_bpe_tokenize")


def build_cli(force=False):
    """The command-line tool over libgtok.so (the reference's gpu_bpe_tokenize modes and output files)."""
    src = os.path.join(HERE, "cli", "gpu_bpe_tokenize.cc")
    if not force and not _newer(CLI, [src, os.path.join(HERE, "..", "include", "gtok.h"), LIB]):
        return CLI
    subprocess.run(["g++", "-std=c++17", "-O2", "-o", CLI, src, "-L" + LIB_DIR, "-l:libgtok.so", "-Wl,-rpath," + LIB_DIR], check=True)
    return CLI


def main():
    force = "--force" in sys.argv
    build_lib(force=force, verbose="-v" in sys.argv)
    build_datagen(force=force)
    build_cli(force=force)
    print(LIB)
    print(DATAGEN)
    print(CLI)


if __name__ == "__main__":
    main()
