"""Compile the CUDA sources of this package for sm_100a and load them with ctypes.

Each ``.cu`` file under this folder is one *module*: it is compiled by nvcc into
one shared library the first time a function of it is asked for, and only then,
so a run compiles what its model and dtype need.  Exported functions are marked
``GG_API`` in the source (``extern "C"``, return an int status); their argument
types are read from the source text, so the Python side never repeats a
signature.

Built libraries live in ``_build/`` beside the sources (kept out of version
control) under a name that carries a hash of source, headers and flags, so a
changed source is rebuilt and a stale library is never loaded.  If that folder
cannot be written, a per-user folder under the system temp dir is used.

There is no fallback: if nvcc is missing or compilation fails, `KernelBuildError`
is raised with the compiler's output.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import re
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from typing import Callable, Dict, List, Optional, Tuple

_HERE = os.path.dirname(os.path.abspath(__file__))

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "--shared", "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]

# GOGGUF_B200_DEBUG=1: the debug build.  Kernels that follow a page table check every index and page id
# before they use it and record a bad one in the status word instead of reading there (common.cuh); the
# libraries of the two builds carry different hashes and live side by side.
# GOGGUF_B200_NVCC_EXTRA: further compiler flags; they take part in the hash
if os.environ.get("GOGGUF_B200_NVCC_EXTRA"):
    NVCC_FLAGS.extend(os.environ["GOGGUF_B200_NVCC_EXTRA"].split())
DEBUG = os.environ.get("GOGGUF_B200_DEBUG", "0") == "1"
if DEBUG:
    NVCC_FLAGS.append("-DGG_DEBUG_BOUNDS")

# module name -> source file (relative to this folder)
MODULES: Dict[str, str] = {
    "elementwise": "elementwise.cu",
    "gemm_plain": "gemm_plain.cu",
    "attention_plain": "attention_plain.cu",
    "sampling": "sampling.cu",
    "gemm_tcgen05": "gemm_tcgen05.cu",
    "attention_fast": "attention_fast.cu",
    "gemm_tcgen05_static": "gemm_tcgen05_static.cu",
    "diagnostics": "diagnostics.cu",
}

_HEADERS = ["common.cuh"]
# further files a module's source includes (they take part in its hash)
_INCLUDES: Dict[str, List[str]] = {
    "attention_fast.cu": ["tma_util.cuh"],
    "gemm_tcgen05.cu": ["tma_util.cuh"],
    "gemm_tcgen05_static.cu": ["gemm_tcgen05.cu", "gemm_tcgen05_static.h", "tma_util.cuh"],
    "diagnostics.cu": ["tma_util.cuh"],
}


class KernelBuildError(RuntimeError):
    pass


class KernelError(RuntimeError):
    """A kernel launcher refused its arguments or CUDA reported an error."""


def _say(msg: str) -> None:
    print(f"[gogguf_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("GOGGUF_B200_NVCC"),
                 os.path.join(os.environ.get("CUDA_HOME", ""), "bin", "nvcc") if os.environ.get("CUDA_HOME") else None,
                 shutil.which("nvcc"),
                 "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise KernelBuildError("nvcc not found (looked at $GOGGUF_B200_NVCC, $CUDA_HOME/bin, PATH, /usr/local/cuda/bin); "
                           "the CUDA kernels of gogguf_b200 cannot be built and there is no fallback")


_build_dir_cache: Optional[str] = None


def _build_dir() -> str:
    global _build_dir_cache
    if _build_dir_cache is not None:
        return _build_dir_cache
    cands = []
    if os.environ.get("GOGGUF_B200_BUILD_DIR"):
        cands.append(os.environ["GOGGUF_B200_BUILD_DIR"])
    cands.append(os.path.join(_HERE, "_build"))
    cands.append(os.path.join(tempfile.gettempdir(), f"gogguf_b200_build_{os.getuid()}"))
    for d in cands:
        try:
            os.makedirs(d, exist_ok=True)
            probe = os.path.join(d, f".w{os.getpid()}_{threading.get_ident()}")
            with open(probe, "w"):
                pass
            os.remove(probe)
            _build_dir_cache = d
            return d
        except OSError:
            continue
    raise KernelBuildError(f"no writable build folder among {cands}")


def _module_hash(src: str) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for f in [src] + _HEADERS + _INCLUDES.get(src, []):
        p = os.path.join(_HERE, f)
        if os.path.isfile(p):
            with open(p, "rb") as fh:
                h.update(fh.read())
    return h.hexdigest()[:16]


def library_path(module: str) -> str:
    src = MODULES[module]
    return os.path.join(_build_dir(), f"gg_{module}_{_module_hash(src)}.so")


def compile_module(module: str, verbose: bool = True) -> str:
    """Compile one module if its library is not there yet; return the library path."""
    if module not in MODULES:
        raise KernelBuildError(f"unknown kernel module {module!r}")
    out = library_path(module)
    if os.path.isfile(out):
        return out
    nvcc = find_nvcc()
    src = os.path.join(_HERE, MODULES[module])
    tmp = f"{out}.{os.getpid()}.tmp"
    cmd = [nvcc] + NVCC_FLAGS + ["-I", _HERE, "-o", tmp, src]
    if verbose:
        _say(f"compiling {MODULES[module]} for sm_100a (first use) ...")
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    done = threading.Event()

    def ticker():
        while not done.wait(10.0):
            if verbose:
                _say(f"... still compiling {MODULES[module]} ({time.time() - t0:.0f} s)")

    th = threading.Thread(target=ticker, daemon=True)
    th.start()
    try:
        log, _ = proc.communicate()
    finally:
        done.set()
    if proc.returncode != 0:
        try:
            os.remove(tmp)
        except OSError:
            pass
        raise KernelBuildError(f"nvcc failed on {MODULES[module]} (exit {proc.returncode}):\n{' '.join(cmd)}\n{log}")
    os.replace(tmp, out)
    if verbose:
        _say(f"compiled {MODULES[module]} in {time.time() - t0:.1f} s -> {out}")
    return out


def compile_all(verbose: bool = True, jobs: int = 4) -> List[str]:
    """Compile every module (used by the build check); a few at a time."""
    from concurrent.futures import ThreadPoolExecutor
    with ThreadPoolExecutor(max_workers=jobs) as ex:
        return list(ex.map(lambda m: compile_module(m, verbose), list(MODULES)))


# ----------------------------------------------------------------------------- signatures
_CTYPES = {
    "int": ctypes.c_int,
    "unsigned": ctypes.c_uint,
    "unsigned int": ctypes.c_uint,
    "uint32_t": ctypes.c_uint,
    "int64_t": ctypes.c_longlong,
    "long long": ctypes.c_longlong,
    "uint64_t": ctypes.c_ulonglong,
    "unsigned long long": ctypes.c_ulonglong,
    "size_t": ctypes.c_size_t,
    "float": ctypes.c_float,
    "double": ctypes.c_double,
    "cudaStream_t": ctypes.c_void_p,
}
_API_RE = re.compile(r"GG_API\s+(\w+)\s*\(([^)]*)\)", re.S)


def parse_signatures(source_text: str) -> Dict[str, List[object]]:
    sigs: Dict[str, List[object]] = {}
    for m in _API_RE.finditer(source_text):
        name, args = m.group(1), m.group(2)
        types: List[object] = []
        args = args.strip()
        if args and args != "void":
            for a in args.split(","):
                a = a.strip()
                if "*" in a:
                    types.append(ctypes.c_void_p)
                    continue
                toks = a.replace("const ", "").split()
                tname = " ".join(toks[:-1]) if len(toks) > 1 else toks[0]
                if tname not in _CTYPES:
                    raise KernelBuildError(f"{name}: cannot map argument type {a!r}")
                types.append(_CTYPES[tname])
        sigs[name] = types
    return sigs


class _Module:
    def __init__(self, name: str):
        self.name = name
        path = compile_module(name)
        self.path = path
        self.lib = ctypes.CDLL(path)
        with open(os.path.join(_HERE, MODULES[name]), "r", encoding="utf-8") as f:
            self.sigs = parse_signatures(f.read())
        self.funcs: Dict[str, Callable] = {}

    def func(self, fname: str) -> Callable:
        f = self.funcs.get(fname)
        if f is None:
            if fname not in self.sigs:
                raise KernelError(f"module {self.name!r} exports no function {fname!r}")
            raw = getattr(self.lib, fname)
            raw.argtypes = self.sigs[fname]
            raw.restype = ctypes.c_int

            def call(*args, _raw=raw, _n=fname):
                global _launches
                _launches += 1
                rc = _raw(*args)
                if rc != 0:
                    raise KernelError(f"{_n} failed: {describe_status(rc)}")

            f = self.funcs[fname] = call
        return f


_launches = 0


def launch_count() -> int:
    """How many launcher calls this process has made (each starts one kernel, a few start two)."""
    return _launches


_loaded: Dict[str, _Module] = {}
_lock = threading.Lock()


def module(name: str) -> _Module:
    m = _loaded.get(name)
    if m is None:
        with _lock:
            m = _loaded.get(name)
            if m is None:
                m = _loaded[name] = _Module(name)
    return m


def kernel(module_name: str, fname: str) -> Callable:
    return module(module_name).func(fname)


_STATUS = {
    -1: "unsupported size or argument (the launcher refused it)",
    -2: "unsupported dtype combination",
    -3: "device is not compute capability 10.x (these kernels are built for sm_100a only)",
    -4: "a bounded wait inside the kernel ran out (see the kernel's status word)",
    -5: "tensor map creation failed",
}


def describe_status(rc: int) -> str:
    if rc in _STATUS:
        return f"{_STATUS[rc]} (status {rc})"
    return f"CUDA error {rc}"
