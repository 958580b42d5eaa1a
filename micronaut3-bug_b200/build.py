"""Builds the native code in-tree: the CUDA library (sm_100a only) and, for the tests, the CPU checker.

    python -m "micronaut3-bug_b200.build"        # or: from the package, build.build_all()

nvcc cross-compiles without a GPU, so this also is the "does it build" check.
"""
from __future__ import annotations

import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
INCLUDE = os.path.join(ROOT, "include")
LIB = os.path.join(PKG, "libpetjson.so")
GEN_LIB = os.path.join(PKG, "libpj_gen.so")
ORACLE_DIR = os.path.join(ROOT, "oracle")
ORACLE_LIB = os.path.join(ORACLE_DIR, "libpj_oracle.so")
FACADE_DEMO = os.path.join(PKG, "host", "object_mapper_demo")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-I", INCLUDE, "-I", CSRC]


def _newer(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def _run(cmd: list[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        raise RuntimeError("build step failed: " + cmd[0])


def _sources(d: str, exts: tuple[str, ...]) -> list[str]:
    return sorted(os.path.join(d, f) for f in os.listdir(d) if f.endswith(exts))


def build_library(force: bool = False, verbose_ptxas: bool = False) -> str:
    deps = _sources(CSRC, (".cu", ".cuh", ".h")) + [os.path.join(INCLUDE, "petjson.h")]
    if not force and _newer(LIB, deps):
        return LIB
    from concurrent.futures import ThreadPoolExecutor

    nvcc = os.environ.get("NVCC", "nvcc")
    extra = ["-Xptxas", "-v"] if verbose_ptxas else []
    api_o = os.path.join(CSRC, "pj_api.o")
    jobs = [[nvcc, *NVCC_FLAGS, *extra, "-c", os.path.join(CSRC, "pj_api.cu"), "-o", api_o]]
    tile_objs = []
    for schema in (1, 2, 3, 4):  # the tile kernel once per model set (Pet, Order, User, mixed), side by side
        obj = os.path.join(CSRC, f"pj_tile_{schema}.o")
        tile_objs.append(obj)
        jobs.append([nvcc, *NVCC_FLAGS, *extra, f"-DPJ_TILE_SCHEMA={schema}", "-c", os.path.join(CSRC, "pj_tile_inst.cu"), "-o", obj])
    with ThreadPoolExecutor(max_workers=len(jobs)) as pool:
        list(pool.map(_run, jobs))
    _run([nvcc, "-shared", "-o", LIB, api_o, *tile_objs, "-ldl", "-lpthread"])
    return LIB


def build_generator(force: bool = False) -> str:
    """The seeded workload generator: host-only C, a library of its own (no CUDA, no link to libpetjson.so)."""
    src = os.path.join(PKG, "gen", "pj_gen.c")
    if not force and _newer(GEN_LIB, [src, os.path.join(INCLUDE, "petjson.h"), os.path.join(INCLUDE, "petjson_gen.h")]):
        return GEN_LIB
    _run(["gcc", "-O2", "-std=c11", "-fPIC", "-shared", "-Wall", "-I", INCLUDE, src, "-o", GEN_LIB, "-lm"])
    return GEN_LIB


def build_oracle(force: bool = False) -> str:
    src = os.path.join(ORACLE_DIR, "pj_oracle.c")
    if not force and _newer(ORACLE_LIB, [src, os.path.join(INCLUDE, "petjson.h")]):
        return ORACLE_LIB
    _run(["gcc", "-O2", "-std=c11", "-fPIC", "-shared", "-Wall", "-Wextra", "-pthread", "-I", INCLUDE, src, "-o", ORACLE_LIB])
    return ORACLE_LIB


def build_facade_demo(force: bool = False) -> str:
    """The C++ mirror of the ObjectMapper surface, compiled into a small self-checking program."""
    src = os.path.join(PKG, "host", "object_mapper_demo.cpp")
    hdr = os.path.join(PKG, "host", "object_mapper.hpp")
    if not os.path.exists(src):
        return ""
    if not force and _newer(FACADE_DEMO, [src, hdr, LIB]):
        return FACADE_DEMO
    _run(["g++", "-O2", "-std=c++17", "-Wall", "-I", INCLUDE, "-I", os.path.join(PKG, "host"), src, "-o", FACADE_DEMO,
          "-L", PKG, "-lpetjson", "-Wl,-rpath," + PKG])
    return FACADE_DEMO


def build_all(force: bool = False) -> None:
    build_library(force)
    build_generator(force)
    build_oracle(force)
    build_facade_demo(force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
    print(LIB)
