"""Link compatibility of libmnemo_b200.so with the reference's host code (no GPU needed).

The reference has no header for its kernel ABI: forward.c re-declares every wrapper (src/forward.c:24-152)
and engine.c calls a few more (src/engine.c:1205, 1530-1533). A drop-in must make those references resolve
to THIS library. The recipe: build the reference's kernels.o / gemm_q4k.o for the symbols
this library does not provide, make the symbols it does provide LOCAL in those objects
(objcopy --localize-symbol), and link with -lmnemo_b200. Weakening the symbols instead does not work: a
weak definition inside the same link still satisfies the references, so the reference kernels keep running.
Both facts are checked on a toy pair of objects; the real recipe is checked on the reference's own sources
when its checkout is available (it is compiled where it lies, into a temporary directory)."""
import os
import re
import shutil
import subprocess
import sys

import pytest

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
LIB_DIR = os.path.join(ROOT, "mnemocuda_b200")
LIB = os.path.join(LIB_DIR, "libmnemo_b200.so")

# the reference's symbols this library defines (include/mnemo_b200.h, Part 1)
OURS = ["cuda_kernels_init", "cuda_matvec_q4k", "cuda_matvec_q4k_add", "cuda_matvec_q4k_qkv", "cuda_matvec_q4k_dual",
        "cuda_matvec_q4k_scaled_add", "cuda_matvec_q6k", "cuda_matvec_f32", "cuda_topk_softmax", "cuda_swiglu",
        "cuda_scaled_add", "cuda_rms_norm", "cuda_rms_norm_residual", "cuda_rms_norm_batched", "cuda_rms_norm_qk",
        "cuda_rope", "cuda_f32_to_f16", "cuda_f32_to_f16_dual", "cuda_attention_f16kv", "cuda_residual_add",
        "cuda_embedding_lookup_q4k", "cuda_sample_token", "cuda_get_rope_kernel_ptr", "cuda_get_f16dual_kernel_ptr",
        "cuda_get_attn_f16kv_kernel_ptr"]
HOT = OURS[:11]


def run(cmd, **kw):
    return subprocess.run(cmd, check=True, capture_output=True, text=True, **kw)


def reference_dir():
    for cand in (os.environ.get("MNEMO_REFERENCE_DIR"), os.path.join(ROOT, "..", "reference")):
        if cand and os.path.isfile(os.path.join(cand, "src", "forward.c")):
            return os.path.abspath(cand)
    return None


def test_library_defines_every_symbol_it_claims():
    out = run(["nm", "-D", "--defined-only", LIB]).stdout
    defined = set(re.findall(r" T (\w+)", out))
    missing = [s for s in OURS if s not in defined]
    assert not missing, missing


def test_localize_routes_calls_to_the_replacement_and_weaken_does_not(tmp_path):
    """Toy: host.o calls hot(); ref.o defines hot() returning 1 (and cold() returning 10); librepl.so defines
    hot() returning 2. Which hot() runs depends on what was done to ref.o before the link."""
    (tmp_path / "host.c").write_text("int hot(void); int cold(void); int call(void) { return hot() + cold(); }\n")
    (tmp_path / "ref.c").write_text("int hot(void) { return 1; } int cold(void) { return 10; }\n")
    (tmp_path / "repl.c").write_text("int hot(void) { return 2; }\n")
    (tmp_path / "main.c").write_text('#include <stdio.h>\nint call(void); int main(void) { printf("%d\\n", call()); return 0; }\n')
    cc = shutil.which("gcc") or "gcc"
    env = dict(os.environ)
    env.pop("CC", None)
    for src in ("host", "ref", "repl"):
        run([cc, "-fPIC", "-c", f"{src}.c", "-o", f"{src}.o"], cwd=tmp_path, env=env)
    run([cc, "-shared", "-o", "librepl.so", "repl.o"], cwd=tmp_path, env=env)
    results = {}
    for how in ("weaken", "localize"):
        run(["objcopy", f"--{how}-symbol=hot", "ref.o", f"ref_{how}.o"], cwd=tmp_path)
        run([cc, "-shared", "-o", f"libengine_{how}.so", "host.o", f"ref_{how}.o", "-L.", "-lrepl", "-Wl,-rpath,$ORIGIN"],
            cwd=tmp_path, env=env)
        run([cc, "main.c", "-o", f"main_{how}", "-L.", f"-lengine_{how}", "-lrepl", "-Wl,-rpath,$ORIGIN"], cwd=tmp_path, env=env)
        results[how] = int(run([str(tmp_path / f"main_{how}")]).stdout.strip())
    assert results["weaken"] == 11, results     # the weak reference definition still wins: NOT a drop-in
    assert results["localize"] == 12, results   # the replacement's hot() runs; cold() still comes from the reference


@pytest.mark.skipif(reference_dir() is None or shutil.which("nvcc") is None,
                    reason="needs the reference checkout (MNEMO_REFERENCE_DIR or ../reference) and nvcc")
def test_reference_host_code_binds_hot_symbols_to_this_library(tmp_path):
    ref = reference_dir()
    src = os.path.join(ref, "src")
    cc = shutil.which("gcc") or "gcc"
    env = dict(os.environ)
    env.pop("CC", None)
    env.pop("CXX", None)
    cuda_inc = os.path.join(os.path.dirname(os.path.dirname(shutil.which("nvcc"))), "include")
    # the reference's host objects, compiled where they lie (flags: reference Makefile:5)
    host_objs = []
    for name in ("forward", "engine", "heat", "io_pool", "tokenizer", "json_helpers"):
        obj = tmp_path / f"{name}.o"
        run([cc, "-O2", "-fPIC", "-w", "-I", cuda_inc, "-I", src, "-c", os.path.join(src, name + ".c"), "-o", str(obj)], env=env)
        host_objs.append(str(obj))
    und = run(["nm", "-u", host_objs[0], host_objs[1]]).stdout
    imported = set(re.findall(r"U ((?:cuda_)\w+)", und))
    imported = {s for s in imported if not s.startswith(("cudaM", "cudaS", "cudaG", "cudaE", "cudaD", "cudaF", "cudaH", "cudaL", "cudaP"))}
    assert set(HOT) - {"cuda_matvec_q4k_scaled_add"} <= imported | {"cuda_matvec_q4k_scaled_add"}
    # the reference's kernel objects, for the symbols this library does not provide
    kobjs = []
    for name in ("kernels", "gemm_q4k"):
        obj = tmp_path / f"{name}.o"
        run(["nvcc", "-O2", "--use_fast_math", "-arch=sm_100", "-Xcompiler", "-fPIC", "-I", src, "-c",
             os.path.join(src, name + ".cu"), "-o", str(obj)], env=env)
        loc = tmp_path / f"{name}_local.o"
        run(["objcopy"] + [f"--localize-symbol={s}" for s in OURS] + [str(obj), str(loc)])
        kobjs.append(str(loc))
    out = tmp_path / "libmnemo_cuda_dropin.so"
    run(["nvcc", "-shared", "-o", str(out)] + host_objs + kobjs + ["-L", LIB_DIR, "-lmnemo_b200", "-lcudart", "-lpthread", "-lm",
        "-Xlinker", "--no-undefined", "-Xlinker", "-rpath," + LIB_DIR], env=env)
    needed = run(["readelf", "-d", str(out)]).stdout
    assert "libmnemo_b200.so" in needed
    undefined = set(re.findall(r"U (\w+)", run(["nm", "-D", "--undefined-only", str(out)]).stdout))
    used = [s for s in OURS if s in imported]
    assert used and all(s in undefined for s in used), [s for s in used if s not in undefined]
    # at load time every one of them binds to this library (eager binding, the dynamic linker's own log)
    env2 = dict(env, LD_DEBUG="bindings", LD_BIND_NOW="1")
    log = subprocess.run([sys.executable, "-c", f"import ctypes; ctypes.CDLL({str(out)!r})"], env=env2, capture_output=True,
                         text=True).stderr
    for s in used:
        m = re.findall(rf"binding file {re.escape(str(out))} \[0\] to (\S+) \[0\]: normal symbol `{s}'", log)
        assert m and all(t.endswith("libmnemo_b200.so") for t in m), (s, m[:2])
    # and the symbols this library does not provide still come from the reference's own objects
    defined = set(re.findall(r" T (\w+)", run(["nm", "-D", "--defined-only", str(out)]).stdout))
    assert {"cuda_matvec_q3k", "cuda_matvec_q5k", "cuda_matvec_q8_0", "cuda_gemm_q4k", "cuda_quantize_mmq_q8_1"} <= defined
