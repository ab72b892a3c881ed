"""CPU-only checks: the oracle's collective semantics, the simulated flag protocol (including a rank
that never arrives), the library's exported symbols, and the peer-table exchange with gloo ranks."""
import ctypes
import os
import subprocess
import sys

import numpy as np

import k3o
from util import normal_bf16, rng

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_rs_sequence_matches_ring_orders():
    assert list(k3o.rs_sequence(1, 4, 6)) == [2, 3, 0, 1]       # peers ascending, own last (the NCCL ring)
    assert list(k3o.rs_sequence(1, 4, 0)) == [1, 2, 3, 0]       # own first
    assert list(k3o.rs_sequence(1, 4, 7)) == [0, 3, 2, 1]       # descending, own last
    assert list(k3o.rs_sequence(0, 1, 0)) == [0]
    for W in (2, 4, 8):
        for order in range(2 * W):
            for r in range(W):
                assert sorted(k3o.rs_sequence(r, W, order)) == list(range(W))


def test_rs_pull_oracle_against_numpy_chain():
    g = rng(11)
    W, count = 4, 4096
    partials = [normal_bf16(g, (W * count,)) for _ in range(W)]
    for rank in range(W):
        seq = k3o.rs_sequence(rank, W, 6)
        a = k3o.bf16_to_f32(partials[seq[0]][rank * count:(rank + 1) * count])
        for k in seq[1:]:
            a = k3o.bf16_to_f32(k3o.f32_to_bf16(a + k3o.bf16_to_f32(partials[k][rank * count:(rank + 1) * count])))
        assert np.array_equal(k3o.rs_pull(partials, rank, 6), k3o.f32_to_bf16(a))


def test_simulated_flag_protocol():
    bad, status = k3o.sim_barrier(4, slots=6, replays=50, units=896)
    assert bad == 0 and not status.any()
    bad, status = k3o.sim_barrier(8, slots=3, replays=20, units=1)
    assert bad == 0


def test_simulated_flag_protocol_absent_rank_times_out_and_reports():
    bad, status = k3o.sim_barrier(4, slots=2, replays=3, units=896, absent_rank=2, timeout_us=20000)
    assert bad == 3
    assert status[2] == 0 and all(status[r] == 1 + 2 for r in (0, 1, 3))    # every waiter names peer 2


def test_library_exports_every_declared_symbol():
    sys.path.insert(0, os.path.join(ROOT, "kern-k3_b200"))
    lib = os.path.join(ROOT, "kern-k3_b200", "lib", "libk3g.so")
    if not os.path.exists(lib):
        import build
        build.build()
    import k3g
    assert len(k3g.PROTOTYPES) >= 30
    handle = ctypes.CDLL(lib)
    for name in k3g.PROTOTYPES:
        assert hasattr(handle, name), name
    # argument checks run before any CUDA call, so they work without a GPU
    assert k3g.raw("k3g_resnorm_mxfp8", None, None, None, None, None, None, None, 1, 7168, 1e-6, 0, None) == -1
    assert k3g.raw("k3g_rs_pull", 16, 16, 16, 12, 0, 0, 1, 1, None) == -2
    assert k3g.raw("k3g_router_topk", 16, 16, 16, 16, 16, 4, 200, 8, None) == -2


def _launchers(k3g):
    """Every declared entry that launches kernels: the set-up helpers (peer memory, wait status, device query) take
    host pointers and are exercised elsewhere."""
    skip = ("k3g_peer_", "k3g_wait_status", "k3g_device_sms")
    return {n: a for n, a in sorted(k3g.PROTOTYPES.items()) if not n.startswith(skip)}


def test_every_launcher_rejects_null_pointers_before_any_cuda_call():
    """All pointers null, every size zero: each launcher must answer K3G_ENULL.  Nothing may reach a launch -- a launch
    attempt would show as a positive cudaError (on a host without a GPU) or as 0."""
    sys.path.insert(0, os.path.join(ROOT, "kern-k3_b200"))
    import k3g
    entries = _launchers(k3g)
    assert len(entries) >= 60
    for name, args in entries.items():
        vals = [None if "*" in ty else (0.0 if "float" in ty else 0) for ty, _ in args]
        assert getattr(k3g.lib, name)(*vals) == -1, name


def test_no_launcher_launches_on_zero_sizes():
    """Non-null, 16-byte aligned pointers (never dereferenced on the host) and every size zero: a launcher either
    rejects the shape or returns 0 for the empty input; none attempts a launch (which would return a positive
    cudaError on a host without a GPU).  kern_k3_fmha_lens has no size argument (one fixed block) and is left out."""
    sys.path.insert(0, os.path.join(ROOT, "kern-k3_b200"))
    import k3g
    for name, args in _launchers(k3g).items():
        if name == "k3g_fmha_lens":
            continue
        vals = [(None if a == "stream" else 4096) if "*" in ty else (0.0 if "float" in ty else 0) for ty, a in args]
        rc = getattr(k3g.lib, name)(*vals)
        assert rc in (0, -2, -4, -5), (name, rc)


def test_host_pipeline_chunks_partition_the_shard_with_a_tapered_tail():
    sys.path.insert(0, os.path.join(ROOT, "kern-k3_b200"))
    from k3g.pipeline import TpGlue
    for rows in (1, 2, 7, 8, 13, 100, 2048, 16384, 16385):
        for chunks in (1, 3, 8, 16):
            b = TpGlue.chunk_bounds(rows, chunks)
            assert b[0][0] == 0 and b[-1][1] == rows
            assert all(x[1] == y[0] for x, y in zip(b, b[1:])) and all(x[1] > x[0] for x in b)
    sizes = [r1 - r0 for r0, r1 in TpGlue.chunk_bounds(16384, 8)]
    assert sizes == [2048] * 7 + [1024, 512, 256, 256]             # the tail nothing overlaps is one small chunk


def test_dropin_cubins_export_reference_entry_names():
    """Every cubin built for a reference module name contains the entry names the manifest launches."""
    cdir = os.path.join(ROOT, "kern-k3_b200", "lib", "cubin")
    want = {
        "k3_residual_v2+LAND_BF16=1": ["kern_k3_attnres_rms", "kern_k3_land_add_attnres_rms", "kern_k3_land_add2"],
        "k3_quant_fp8_pair_v2": ["kern_quant_fp8_amax_v2", "kern_quant_fp8_apply_v2", "kern_k3_moe_quant"],
        "k3_router_argmax": ["kern_k3_router_topk"],
        "k3_reducescatter_pull_nr4": ["kern_k3_rs_pull", "kern_k3_rs_arrive1", "kern_k3_allgather4_push", "kern_k3_epoch_bump", "kern_k3_flags_init"],
        "k3_mla_prep_v2+INNER=3072+MLA_FUSED=5184": ["kern_k3_mla_prep_head", "kern_k3_mla_prep_gate"],
        "k3_span_gather_v3+HEADS=24": ["kern_k3_span_gather", "kern_k3_kda_out_gate"],
    }
    for mod, entries in want.items():
        path = os.path.join(cdir, mod + ".cubin")
        assert os.path.exists(path), path
        blob = open(path, "rb").read()
        for e in entries:
            assert e.encode() in blob, (mod, e)


def test_peer_group_exchange_with_gloo_ranks():
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                        "--master-port", "29533", os.path.join(ROOT, "tests", "gloo_worker.py")], capture_output=True, text=True, timeout=300)
    sys.stdout.write(r.stdout[-3000:]); sys.stderr.write(r.stderr[-3000:])
    assert r.returncode == 0 and r.stdout.count("GLOO_OK") == 2


def test_header_is_plain_c_and_links_from_a_c_program(tmp_path):
    """include/k3g.h must be usable from C (what cgo / JNI / any FFI binds): compile a C translation unit that
    takes the address of every declared entry point with gcc and link it against libk3g.so.  Nothing is launched;
    the argument-validation path is exercised with a null pointer (rejected before any CUDA call)."""
    import shutil
    import subprocess
    import k3g
    if shutil.which("gcc") is None:
        pytest.skip("gcc not available")
    names = sorted(k3g.PROTOTYPES)
    src = tmp_path / "abi.c"
    src.write_text('#include "k3g.h"\n#include <stdio.h>\n'
                   "static void* table[] = {%s};\n" % ", ".join("(void*)%s" % n for n in names) +
                   "int main(void) {\n"
                   "  int rc = k3g_moe_quant(0, 0, 0, 1, 32, 0, 0);          /* null input: K3G_ENULL, no launch */\n"
                   '  printf("%d %d\\n", (int)(sizeof table / sizeof table[0]), rc);\n'
                   "  return 0;\n}\n")
    exe = tmp_path / "abi"
    libdir = os.path.dirname(k3g.LIB_PATH)
    subprocess.check_call(["gcc", "-std=c99", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe),
                           "-L", libdir, "-lk3g", "-Wl,-rpath," + libdir])
    out = subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split()
    assert int(out[0]) == len(names) and int(out[1]) == -1


def test_bench_reference_arm_prints_the_contract_line():
    """`bench.py --impl reference` runs on the host cores alone (no GPU): one JSON line with the contract's keys, the same
    `config` object the GPU arm prints, the requested step / warm-up counts honoured, and a CPU baseline that names its
    sample."""
    import json
    import subprocess
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "2", "--warmup", "1"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    for k in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "vs_baseline", "dtype", "data",
              "config", "cpu_baseline", "e2e", "gpu_launches"):
        assert k in d, k
    assert d["impl"] == "reference" and d["steps"] == 2 and d["warmup"] == 1 and d["n_gpus"] == 2 and d["higher_is_better"] is False
    assert d["config"]["world"] == 2 and d["config"]["tokens"] == 16384 and "config1" in d["config"]["workload"]
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1 and "world 2" in d["cpu_baseline"]["sample"]
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["value"] == d["value"] > 0
    sys.path.insert(0, ROOT)
    import bench
    assert bench.workload_config(2) == d["config"]                # what the GPU arm prints for the same world
