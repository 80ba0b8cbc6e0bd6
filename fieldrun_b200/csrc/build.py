"""Compiles the CUDA sources of this folder for sm_100a into shared libraries, one per group of kernels.

A group holds the kernels that are needed together (``GROUPS``): a model asks for the groups of its parts, and only
those are compiled, all their sources side by side, the first time they are needed.  The libraries are kept beside the
sources (``_build/``), or in a per-user temporary folder when the checkout cannot be written.  A library's file name
carries a hash of its sources, the headers and the flags, so a changed source never runs stale code.  There is no
fallback: without nvcc or with a failing compile the error is raised.
"""
from __future__ import annotations

import concurrent.futures
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time

HERE = os.path.dirname(os.path.abspath(__file__))
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
              "-Xcompiler", "-fvisibility=hidden"]


class BuildError(RuntimeError):
    pass


# Which sources make which library.  Every library also gets errors.cu (the error text of its entry points).
GROUPS: dict[str, tuple[str, ...]] = {
    "common": ("elementwise.cu", "layernorm.cu", "attention_generic.cu", "sampling.cu", "stream_ops.cu", "token_inputs.cu",
               "sandwich_norm.cu"),
    "attention": ("attention_mma.cu", "attention_decode_tma.cu", "attention_tc.cu"),
    "streams": ("experts_stream.cu", "experts_mma.cu"),
    "experts": ("routing.cu", "experts_generic.cu"),
    "products": ("experts_tc.cu",),
    "recurrent": ("gla.cu",),
    "scans": ("scans.cu",),
    "delta": ("delta_rule.cu",),
    "latent": ("latent_attention.cu", "latent_attention_tc.cu"),
    "extras": ("attention_decode_noalloc.cu", "wait_probe.cu"),
}
SHARED_SOURCE = "errors.cu"


def sources(group: str | None = None) -> list[str]:
    """The sources of one group (with the shared one), or every ``.cu`` file of the folder."""
    if group is None:
        return sorted(f for f in os.listdir(HERE) if f.endswith(".cu"))
    return sorted(GROUPS[group] + (SHARED_SOURCE,))


def check_groups() -> None:
    """Every source belongs to exactly one group."""
    listed = [name for names in GROUPS.values() for name in names] + [SHARED_SOURCE]
    if sorted(listed) != sources():
        raise BuildError(f"the groups name {sorted(listed)}, the folder holds {sources()}")


def _headers() -> list[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith((".cuh", ".h")))


def _nvcc() -> str:
    for candidate in (os.environ.get("FIELDRUN_B200_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and os.path.isfile(candidate):
            return candidate
    raise BuildError("nvcc was not found (looked at $FIELDRUN_B200_NVCC, PATH and /usr/local/cuda/bin); "
                     "the CUDA kernels of fieldrun_b200 cannot be built and there is no other path")


def source_hash(group: str) -> str:
    h = hashlib.sha256()
    for name in sources(group) + _headers():
        h.update(name.encode())
        with open(os.path.join(HERE, name), "rb") as handle:
            h.update(handle.read())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def _build_dir() -> str:
    override = os.environ.get("FIELDRUN_B200_BUILD_DIR")
    candidates = [override] if override else []
    candidates.append(os.path.join(HERE, "_build"))
    candidates.append(os.path.join(tempfile.gettempdir(), f"fieldrun_b200_build_{os.getuid()}"))
    for path in candidates:
        try:
            os.makedirs(path, exist_ok=True)
            probe = os.path.join(path, f".write_probe_{os.getpid()}")
            with open(probe, "w"):
                pass
            os.remove(probe)
            return path
        except OSError:
            continue
    raise BuildError(f"no writable folder for the compiled kernels among {candidates}")


def library_path(group: str, create_dir: bool = True) -> str:
    tag = source_hash(group)
    in_tree = os.path.join(HERE, "_build", f"libfieldrun_b200_{group}_{tag}.so")
    if os.path.isfile(in_tree) or not create_dir:
        return in_tree
    return os.path.join(_build_dir(), f"libfieldrun_b200_{group}_{tag}.so")


def _say(message: str) -> None:
    print(f"[fieldrun_b200] {message}", file=sys.stderr, flush=True)


def build(groups=None, verbose: bool = True, ptxas_info: bool = False) -> dict[str, str]:
    """Compile what is missing of ``groups`` (default: all of them), every source of every missing library side by
    side, and return group -> path of its shared library."""
    check_groups()
    groups = list(GROUPS) if groups is None else list(dict.fromkeys(groups))
    targets = {group: library_path(group) for group in groups}
    missing = [group for group in groups if not os.path.isfile(targets[group])]
    if not missing:
        return targets
    nvcc = _nvcc()
    started = time.time()
    jobs = [(group, name) for group in missing for name in sources(group)]
    if verbose:
        _say(f"compiling {len(jobs)} CUDA sources for sm_100a ({', '.join(missing)}) into {os.path.dirname(targets[missing[0]])} "
             f"(first use; takes a minute or two)")

    def compile_one(job: tuple[str, str]) -> tuple[str, str, str]:
        group, name = job
        out_dir = os.path.dirname(targets[group])
        obj = os.path.join(out_dir, f"{group}_{name[:-3]}_{source_hash(group)}_{os.getpid()}.o")
        cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", HERE, "-c", os.path.join(HERE, name), "-o", obj]
        if ptxas_info:
            cmd[1:1] = ["-Xptxas", "-v"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise BuildError(f"nvcc failed on {name}:\n{proc.stdout}\n{proc.stderr}")
        return group, obj, proc.stderr

    objects: dict[str, list[str]] = {group: [] for group in missing}
    logs: list[str] = []
    workers = max(1, min(len(jobs), os.cpu_count() or 1))
    with concurrent.futures.ThreadPoolExecutor(max_workers=workers) as pool:
        futures = {pool.submit(compile_one, job): job for job in jobs}
        done = 0
        for future in concurrent.futures.as_completed(futures):
            group, obj, log = future.result()
            objects[group].append(obj)
            logs.append(log)
            done += 1
            if verbose:
                _say(f"  compiled {futures[future][1]} for {group} ({done}/{len(jobs)}, {time.time() - started:.0f} s)")
    for group in missing:
        target = targets[group]
        partial = target + f".tmp{os.getpid()}"
        link = [nvcc, *ARCH_FLAGS, "-shared", "-o", partial, *sorted(objects[group]), "-lcudart"]
        proc = subprocess.run(link, capture_output=True, text=True)
        if proc.returncode != 0:
            raise BuildError(f"linking the kernels of {group} failed:\n{proc.stdout}\n{proc.stderr}")
        os.replace(partial, target)
        out_dir = os.path.dirname(target)
        prefix = f"libfieldrun_b200_{group}_"
        for name in os.listdir(out_dir):                    # libraries of older sources, and the single library of before
            stale_group = name.startswith(prefix) and name.endswith(".so") and name != os.path.basename(target)
            stale_single = name.startswith("libfieldrun_b200_") and name.endswith(".so") and name.count("_") == 2
            if stale_group or stale_single:
                try:
                    os.remove(os.path.join(out_dir, name))
                except OSError:
                    pass
        for obj in objects[group]:
            try:
                os.remove(obj)
            except OSError:
                pass
    if verbose:
        _say(f"built {', '.join(os.path.basename(targets[g]) for g in missing)} in {time.time() - started:.0f} s")
    if ptxas_info:
        sys.stderr.write("\n".join(logs))
    return targets


if __name__ == "__main__":
    for _group, _path in build(ptxas_info="--ptxas" in sys.argv).items():
        print(_group, _path)
