#!/usr/bin/env python
"""Round benchmark: batch-1 decode of a Llama-2-7B-shaped Q4_K_M model at 4k context on B200 (BASELINE.json configs[1]).

One "step" = one decoded token = one pass of the hot path (all MUL_MATs as decode GEMVs + FLASH_ATTN_EXT over the f16 KV
cache + the small ops of the graph) through the ggml_backend boundary of libkcpp_b200.so.

Legs (all printed in ONE JSON line by rank 0):
  value      tokens/s with everything resident in HBM: graph_compute replayed K times, CUDA events on the backend stream.
  e2e        tokens/s through the public call b200_llama_decode with HOST buffers: per step host token id -> H2D (token,
             position, KQ mask), graph_compute, D2H of the logits (pinned), host argmax feeds the next token (greedy).
  roofline   the decode GEMV family: the token's GEMV launch sequence (same types, shapes and order, rotating weight sets
             larger than L2) timed alone with CUDA events; achieved = algorithmic bytes / time against the measured HBM peak.
  e2e_llamacpp  the same metric with the REFERENCE's unmodified llama.cpp as the host: llama_decode under ggml_backend_sched with
             libkcpp_b200.so attached by ggml_backend_register, on a GGUF file of the workload (tools/make_gguf.py).
  cpu_baseline  the reference's own llama.cpp + CPU backend (oracle/_ref) decoding the same GGUF on this box's host cores
             (bounded sample: 16 tokens at n_kv = 4096).
  tp_70b     auxiliary: BASELINE.json configs[4], ONE Llama-3-70B-shaped Q4_K_M model sharded over all N ranks (strong scaling,
             NCCL all-reduce / all-gather in the captured graph); at N = 1 the same model on one GPU, so 1 -> N speed-up is
             the ratio of the tp_70b values of two runs.
`--impl reference` prints the CPU arm only.   N > 1: the headline legs run one 7B replica per rank (weak scaling, no data-path
collective: the 7B model does not need sharding); the sharded path is the tp_70b leg.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOAD = "llama2-7b-q4_k_m"
N_CTX = 4096
N_PREFILLED = 3968  # tg128 at 4k context: cells [0, 3968) pre-filled, positions 3968..4095 decoded (n_kv = 4096 throughout)
PP_BATCH = 512     # auxiliary leg: pp512 prefill of the same model (tensor-core GEMM + multi-column flash attention)
METRIC = "decode_tokens_per_s"
UNIT = "tok/s"


def peaks() -> tuple[float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
        except Exception:
            pass
    return 6650.0, "fallback (B200_PROFILING.md)"


class ClockSampler:
    """nvidia-smi clocks / throttle reasons during the timed region (B200_PROFILING.md recipe)."""
    Q = "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index: int):
        self.rows: list[list[str]] = []
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(index)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
                for n, v in zip(names, r[3:7]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            except Exception:
                continue
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------------ llama.cpp-level legs
# The reference's own, unmodified llama.cpp (oracle/_ref/libllama_ref*.so + llama_harness, compiled from /root/reference by
# oracle/Makefile; the binaries travel to the GPU box) decodes the SAME GGUF file: on its CPU backend (reference arm,
# cpu_baseline) and with libkcpp_b200.so attached through ggml_backend_register (e2e_llamacpp).
def _cpu_flags() -> set:
    try:
        for line in open("/proc/cpuinfo"):
            if line.startswith("flags"):
                return set(line.split(":", 1)[1].split())
    except OSError:
        pass
    return set()


def harness_path():
    ref = ROOT / "oracle" / "_ref"
    if {"avx512f", "avx512bw", "avx512vl", "avx512dq", "avx512_vnni"} <= _cpu_flags() and (ref / "llama_harness_avx512").exists():
        return ref / "llama_harness_avx512", "avx512-vnni build"
    return (ref / "llama_harness"), "avx2 build"


def host_threads() -> int:
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return os.cpu_count() or 1


def bench_gguf(shape) -> Path:
    """The workload as a GGUF file (gguf-py writer, tools/make_gguf.py): the configuration's shapes and llama_tensor_get_type mix
    with random-init quantised blocks (throughput runs need no trained or even reference-quantised values)."""
    d = Path(os.environ.get("B200_GGUF_CACHE", "/tmp/b200_gguf"))
    d.mkdir(parents=True, exist_ok=True)
    out = d / f"bench_{shape.name}.gguf"
    if not out.exists():
        sys.path.insert(0, str(ROOT / "tools"))
        import make_gguf
        tmp = out.with_suffix(".tmp")
        make_gguf.build(shape, tmp, None, seed=1234, replicate_layers=True)
        tmp.rename(out)
    return out


def run_harness(model: Path, backend: str, extra: list, timeout: float = 900.0) -> dict:
    exe, build = harness_path()
    if not exe.exists():
        raise FileNotFoundError(f"{exe} missing (built by oracle/Makefile where /root/reference exists)")
    cmd = [str(exe), "--model", str(model), "--quiet", "--n-ctx", str(N_CTX)] + [str(x) for x in extra]
    if backend == "b200":
        cmd += ["--backend-lib", str(ROOT / "koboldcpp_b200" / "libkcpp_b200.so")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout)
    if r.returncode != 0:
        raise RuntimeError(f"llama_harness rc={r.returncode}: {r.stderr[-600:]}")
    j = json.loads(r.stdout.strip().splitlines()[-1])
    j["build"] = build
    return j


def llamacpp_cpu_decode(shape, n_gen: int, n_warm: int) -> dict:
    """tg at n_kv = 4096 through llama_decode on the reference CPU backend with all host threads.  The KV cache is brought to
    N_PREFILLED occupied cells by the harness (--kv-fill: the prompt's rows repeated through the reference's own session-state
    format) instead of a 3968-token CPU prompt (~15 tok/s: minutes); the timed decode steps are the real thing."""
    thr = host_threads()
    j = run_harness(bench_gguf(shape), "cpu", ["--n-prompt", 32, "--kv-fill", N_PREFILLED, "--n-gen", n_gen, "--n-warm", n_warm, "--threads", thr])
    return {"tok_s": j["tg_tok_s"], "ms_per_token": 1e3 / j["tg_tok_s"], "cores": j["threads"],
            "sample": f"reference llama.cpp + ggml CPU backend ({j['build']}), llama_decode on the same GGUF, {j['n_gen']} greedy tokens timed after {n_warm} warm-up "
                      f"at n_kv={N_CTX} (KV filled to {N_PREFILLED} cells via llama_state_set_data), {j['threads']} threads"}


def reference_arm(args, rank: int) -> int:
    """The reference's own CPU implementation of the path on this box's host cores: its llama.cpp + ggml CPU backend."""
    if rank != 0:
        return 0
    from koboldcpp_b200.llama import SHAPES
    shape = SHAPES[WORKLOAD]
    try:
        r = llamacpp_cpu_decode(shape, max(4, min(args.steps, 160)), max(1, min(args.warmup, 8)))
    except Exception as ex:  # the harness is prebuilt in oracle/_ref; fall back to the per-layer sample of the same backend
        sys.path.insert(0, str(ROOT / "tests"))
        import cpu_baseline as B
        r = B.time_decode(shape, N_CTX, budget_s=min(150.0, max(10.0, 1.0 * (args.steps + args.warmup))))
        r["sample"] += f" [llama.cpp harness unavailable: {ex}]"
    line = {"impl": "reference", "metric": METRIC, "value": r["tok_s"], "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": r["ms_per_token"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8 dot / f32 accumulate",
            "data": "synthetic", "config": config_dict(shape),
            "cpu_baseline": {"value": r["tok_s"], "unit": UNIT, "cores": r["cores"], "kind": "reference", "sample": r["sample"]},
            "e2e": {"value": r["tok_s"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))
    return 0


def config_dict(shape) -> dict:
    return {"workload": f"{shape.name} random-init GGUF-shaped model, batch-1 greedy decode (tg128) at n_kv={N_CTX} (KV pre-filled to {N_PREFILLED}), f16 KV, flash attention",
            "n_embd": shape.n_embd, "n_layer": shape.n_layer, "n_head": shape.n_head, "n_ff": shape.n_ff, "n_vocab": shape.n_vocab,
            "l2_policy": "inputs larger than L2: 4.0 GB of weights + 2.1 GB of KV streamed per step vs 126 MB L2"}


# ------------------------------------------------------------------------------------------------ GEMV roofline leg
def gemv_launch_plan(shape):
    """The decode GEMV launches of one token as graph_compute issues them (backend_graph.cu: siblings reading the same
    activation are one multi-job launch; two K-quant weight types may share it).  Returns per layer a list of
    (K, [(type, M), ...])."""
    from koboldcpp_b200.llama import tensor_shape, tensor_types
    types = tensor_types(shape)
    kq = {12, 13, 14} if os.environ.get("B200_MIXED_TYPES") else set()  # the planner's opt-in rule (backend_graph.cu: g_mixed_types)
    layers = []
    for il in range(shape.n_layer):
        p = f"blk.{il}."
        launches = []
        for group in (["attn_q.weight", "attn_k.weight", "attn_v.weight"], ["attn_output.weight"], ["ffn_gate.weight", "ffn_up.weight"], ["ffn_down.weight"]):
            K = tensor_shape(shape, p + group[0])[0]
            members = [(types[p + leaf], tensor_shape(shape, p + leaf)[1]) for leaf in group]
            tys = []
            for ty, _ in members:
                if ty not in tys:
                    tys.append(ty)
            if len(tys) == 1 or (len(tys) == 2 and set(tys) <= kq):
                launches.append((K, members))
            else:
                for ty in tys:
                    launches.append((K, [(t, M) for (t, M) in members if t == ty]))
        layers.append(launches)
    head = (shape.n_embd, [(types["output.weight"], shape.n_vocab)])
    return layers, head


def gemv_leg(shape, steps: int, warmup: int) -> dict:
    """Time the token's GEMV sequence alone: weights rotate through 4 layer-sized sets (> L2 between reuses)."""
    import koboldcpp_b200.host as H
    from koboldcpp_b200.lib import GemvJob, check, lib, row_size
    L = lib()
    layers, head = gemv_launch_plan(shape)
    n_sets = 4
    rng = np.random.default_rng(0)
    kinds = sorted({(K, tuple(mem)) for lay in layers for (K, mem) in lay} | {(head[0], tuple(head[1]))})
    pool = {}
    for (K, mem) in kinds:
        sets = []
        for _ in range(1 if (K, list(mem)) == (head[0], list(head[1])) else n_sets):
            sets.append([H.DeviceBuffer.from_numpy(rng.integers(0, 256, size=row_size(ty, K) * M, dtype=np.uint8), pad=256) for (ty, M) in mem])
        pool[(K, mem)] = sets
    kmax = max(k for k, _ in kinds)
    mmax = max(sum(M for _, M in mem) for _, mem in kinds)
    x = H.DeviceBuffer.from_numpy(rng.standard_normal(kmax).astype(np.float32))
    y = H.DeviceBuffer(4 * mmax + 256)
    st = C.c_void_p()
    check(L.b200_stream_create(C.byref(st)))
    L.b200_set_pdl(1)
    alg_bytes = 0
    n_launch = 0

    def issue():
        nonlocal alg_bytes, n_launch
        alg_bytes = 0
        n_launch = 0
        seq = [(il, l) for il, lay in enumerate(layers) for l in lay] + [(0, head)]
        for il, (K, mem) in seq:
            sets = pool[(K, tuple(mem))]
            bufs = sets[il % len(sets)]
            ty0 = mem[0][0]
            rs = row_size(ty0, K)
            if len(mem) == 1:
                check(L.b200_mul_mat_vec_q(ty0, bufs[0].ptr, rs, x.ptr, K, y.ptr, mem[0][1], K, mem[0][1], 1, st))
            else:
                jobs = (GemvJob * len(mem))()
                off = 0
                for j, (ty, M) in enumerate(mem):
                    jobs[j].W = bufs[j].ptr; jobs[j].X = x.ptr; jobs[j].dst = y.ptr + 4 * off; jobs[j].M = M; jobs[j].id_index = -1
                    jobs[j]._pad = ty if ty != ty0 else 0
                    off += M
                check(L.b200_mul_mat_vec_q_multi(ty0, jobs, len(mem), rs, K, off, K, 1, None, 0, 0, st))
            alg_bytes += sum(row_size(ty, K) * M + 4 * M for (ty, M) in mem) + 4 * K
            n_launch += 1

    check(L.b200_graph_begin_capture(st))
    issue()
    g = C.c_void_p()
    check(L.b200_graph_end_capture(st, C.byref(g)))
    for _ in range(max(3, warmup)):
        check(L.b200_graph_launch(g, st))
    check(L.b200_stream_synchronize(st))
    e0, e1 = C.c_void_p(), C.c_void_p()
    check(L.b200_event_create(C.byref(e0))); check(L.b200_event_create(C.byref(e1)))
    check(L.b200_event_record(e0, st))
    for _ in range(steps):
        check(L.b200_graph_launch(g, st))
    check(L.b200_event_record(e1, st))
    ms = C.c_float()
    check(L.b200_event_elapsed_ms(e0, e1, C.byref(ms)))
    L.b200_graph_destroy(g)
    L.b200_set_pdl(0)
    per_token_ms = ms.value / steps
    for sets in pool.values():
        for bufs in sets:
            for b in bufs:
                b.free()
    x.free(); y.free()
    L.b200_stream_destroy(st)
    return {"ms_per_token": per_token_ms, "launches_per_token": n_launch, "alg_bytes_per_token": alg_bytes,
            "avg_launch_us": per_token_ms * 1e3 / n_launch, "gbs": alg_bytes / per_token_ms / 1e6}


# ------------------------------------------------------------------------------------------------ 70B tensor-parallel leg
TP_WORKLOAD = "llama3-70b-q4_k_m"


def tp_leg(rank: int, world: int, local_rank: int, dist, steps: int, warmup: int) -> dict:
    """BASELINE.json configs[4]: Llama-3-70B-shaped Q4_K_M, ONE model sharded over all `world` ranks (strong scaling): q/k/v, gate/up
    and the head split by rows (whole heads per rank), attn_output / ffn_down split along K with one NCCL all-reduce each, the
    logits all-gathered (koboldcpp_b200/tp.py, csrc/comm.cu).  world == 1 is the same model on one GPU (42 GB of weights).
    Timed like the main legs: resident replay with CUDA events on the backend stream, and the public call with host tokens in /
    host logits out; max over ranks."""
    import koboldcpp_b200.llama as LL
    from koboldcpp_b200 import tp
    from koboldcpp_b200.lib import F16, check, lib
    L = lib()
    shape = LL.SHAPES[TP_WORKLOAD]
    t0 = time.time()
    if world > 1:
        tp.comm_init_from_torch(rank, world)
    m = LL.LlamaModel(shape, N_CTX, F16, main_device=local_rank, tp_rank=rank, tp_world=world)
    m.init_random(seed=4321)            # same stream on every rank: each keeps its shard of the same model
    m.finalize(max_batch=PP_BATCH)
    m.kv_fill_random(N_PREFILLED, seed=11)
    setup_s = time.time() - t0
    span = N_CTX - N_PREFILLED
    stream = m.stream
    ev = [C.c_void_p() for _ in range(4)]
    for e in ev:
        check(L.b200_event_create(C.byref(e)))

    def barrier():
        if dist is not None:
            import torch
            torch.cuda.synchronize()
            dist.barrier()
        m.synchronize()

    tok = 1
    for i in range(warmup):
        tok = int(np.argmax(m.decode([tok], N_PREFILLED + i % span)[0]))
    barrier()
    check(L.b200_event_record(ev[0], stream))
    t1 = time.perf_counter()
    for i in range(steps):
        tok = int(np.argmax(m.decode([tok], N_PREFILLED + (warmup + i) % span)[0]))
    check(L.b200_event_record(ev[1], stream))
    ms = C.c_float()
    check(L.b200_event_elapsed_ms(ev[0], ev[1], C.byref(ms)))
    e2e_ms = max(ms.value, (time.perf_counter() - t1) * 1e3)
    st = m.stats()
    barrier()
    for _ in range(warmup):
        m.replay()
    barrier()
    check(L.b200_event_record(ev[2], stream))
    for _ in range(steps):
        m.replay()
    check(L.b200_event_record(ev[3], stream))
    check(L.b200_event_elapsed_ms(ev[2], ev[3], C.byref(ms)))
    res_ms = ms.value
    barrier()
    pp_tokens = [(i * 7919) % shape.n_vocab for i in range(PP_BATCH)]
    pp_ms = []
    for _ in range(3):
        barrier()
        t2 = time.perf_counter()
        m.decode(pp_tokens, 0)
        pp_ms.append((time.perf_counter() - t2) * 1e3)
    pp_best = min(pp_ms[1:])
    if dist is not None:
        import torch
        t = torch.tensor([res_ms, e2e_ms, pp_best], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        res_ms, e2e_ms, pp_best = float(t[0]), float(t[1]), float(t[2])
    m.close()
    if world > 1:
        tp.comm_destroy()
    peak, _ = peaks()
    alg = LL.weight_bytes_per_token(shape) + LL.kv_bytes_per_token(shape, N_CTX, F16)
    return {"workload": f"{shape.name} random-init, batch-1 greedy decode at n_kv={N_CTX}, f16 KV; ONE model over {world} GPU(s)",
            "parallelism": f"tp{world}" if world > 1 else "single", "scaling": "strong", "steps": steps, "warmup": warmup,
            "value": steps / (res_ms / 1e3), "unit": UNIT, "ms_per_step": res_ms / steps,
            "e2e": {"value": steps / (e2e_ms / 1e3), "unit": UNIT, "ms_per_step": e2e_ms / steps},
            "pp512_tokens_per_s": PP_BATCH / (pp_best / 1e3), "pp512_ms": pp_best,
            "alg_bytes_per_step": alg, "hbm_frac_of_aggregate_peak": alg / (res_ms / steps) / 1e6 / (peak * world),
            "launches_per_step": int(st["n_kernels"]), "collectives_per_step": (2 * shape.n_layer + 1) if world > 1 else 0, "setup_s": setup_s}


# ------------------------------------------------------------------------------------------------ product arm
def product_arm(args, rank: int, world: int, local_rank: int) -> int:
    import koboldcpp_b200.llama as LL
    from koboldcpp_b200.lib import F16, check, lib
    L = lib()
    if L.b200_device_count() <= 0:
        print("bench.py: no CUDA device and the product has no CPU path", file=sys.stderr)
        return 2
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist_
        torch.cuda.set_device(local_rank)
        dist_.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        dist = dist_
    check(L.b200_set_device(local_rank), "set_device")
    if os.environ.get("B200_BENCH_ONLY_TP70"):  # developer shortcut: the sharded 70B leg alone (not a round bench line)
        tp70 = tp_leg(rank, world, local_rank, dist, min(args.steps, 32), 3)
        if rank == 0:
            print(json.dumps({"tp_70b_only": tp70}))
        if dist is not None:
            dist.barrier()
            dist.destroy_process_group()
        return 0
    shape = LL.SHAPES[WORKLOAD]
    steps, warmup = args.steps, max(3, args.warmup)
    t_setup = time.time()
    m = LL.LlamaModel(shape, N_CTX, F16, main_device=local_rank)
    m.init_random(seed=1234 + rank)
    m.finalize(max_batch=PP_BATCH)
    m.kv_fill_random(N_PREFILLED, seed=7 + rank)
    setup_s = time.time() - t_setup
    span = N_CTX - N_PREFILLED  # positions cycle inside [3968, 4096): n_kv stays 4096 for any K

    def pos(i):
        return N_PREFILLED + (i % span)

    ev = [C.c_void_p() for _ in range(4)]
    for e in ev:
        check(L.b200_event_create(C.byref(e)))
    stream = m.stream

    def barrier():
        if dist is not None:
            import torch
            torch.cuda.synchronize()
            dist.barrier()
        m.synchronize()

    # ---- e2e leg: the public call with host buffers, greedy token feedback
    tok = 1
    for i in range(warmup):
        tok = int(np.argmax(m.decode([tok], pos(i))[0]))
    barrier()
    clocks = ClockSampler(local_rank)
    check(L.b200_event_record(ev[0], stream))
    t0 = time.perf_counter()
    for i in range(steps):
        tok = int(np.argmax(m.decode([tok], pos(warmup + i))[0]))
    check(L.b200_event_record(ev[1], stream))
    ms = C.c_float()
    check(L.b200_event_elapsed_ms(ev[0], ev[1], C.byref(ms)))
    e2e_wall_ms = (time.perf_counter() - t0) * 1e3
    e2e_ms = max(ms.value, e2e_wall_ms)  # host-synchronous loop: the wall clock bounds the device span from above
    st = m.stats()
    barrier()

    # ---- resident leg: graph_compute replayed with inputs in HBM
    for _ in range(warmup):
        m.replay()
    barrier()
    check(L.b200_event_record(ev[2], stream))
    for _ in range(steps):
        m.replay()
    check(L.b200_event_record(ev[3], stream))
    check(L.b200_event_elapsed_ms(ev[2], ev[3], C.byref(ms)))
    res_ms = ms.value
    clk = clocks.stop()
    barrier()

    # ---- auxiliary leg: pp512 through the same public call (host tokens in, last-token logits out)
    pp_tokens = [(i * 7919) % shape.n_vocab for i in range(PP_BATCH)]
    pp_ms = []
    for _ in range(4):
        t1 = time.perf_counter()
        m.decode(pp_tokens, 0)
        pp_ms.append((time.perf_counter() - t1) * 1e3)
    pp_best = min(pp_ms[1:])
    barrier()

    if dist is not None:
        import torch
        t = torch.tensor([res_ms, e2e_ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        res_ms, e2e_ms = float(t[0]), float(t[1])
    m.close()

    tp70 = None
    if not args.no_tp70:
        try:
            tp70 = tp_leg(rank, world, local_rank, dist, min(steps, 32), 3)
        except Exception as ex:  # the auxiliary leg must not hide the headline numbers
            tp70 = {"error": f"{type(ex).__name__}: {ex}"}

    if rank == 0:
        peak, peak_src = peaks()
        g = gemv_leg(shape, steps, warmup)
        # DRAM bytes per launch from the committed ncu --set full capture (measured / algorithmic ratio of the same kernels)
        traffic, traffic_src = None, None
        try:
            tj = json.loads((ROOT / "profiles" / "ncu_traffic.json").read_text())
            traffic = float(tj["gemv_dram_bytes_over_algorithmic_bytes"]) * g["alg_bytes_per_token"] / g["launches_per_token"]
            traffic_src = "profiles/ncu_traffic.json"
        except Exception:
            pass
        wbytes = LL.weight_bytes_per_token(shape)
        kvbytes = LL.kv_bytes_per_token(shape, N_CTX, F16)
        tok_s = world * steps / (res_ms / 1e3)
        e2e_tok_s = world * steps / (e2e_ms / 1e3)
        # per step: token id + position + ONE mask element (the cell that becomes visible); the decoder re-sends the whole
        # 4 * n_kv * 32-byte mask only when the position does not follow the previous one, i.e. when pos() wraps (every `span` steps)
        wraps = sum(1 for i in range(steps) if pos(warmup + i) != pos(warmup + i - 1) + 1)
        mask_bytes = 4 + (4 * N_CTX * 32 * wraps) // steps
        line = {
            "metric": METRIC, "value": tok_s, "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": res_ms / steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8 dot (dp4a) / f32 accumulate; f16 KV",
            "data": "synthetic", "config": config_dict(shape),
            "e2e": {"value": e2e_tok_s, "unit": UNIT, "h2d_bytes_per_step": 4 + 4 + mask_bytes, "d2h_bytes_per_step": 4 * shape.n_vocab,
                    "ms_per_step": e2e_ms / steps},
            "gpu_launches": int(st["n_kernels"]) * steps * 2,
            "launches_per_step": int(st["n_kernels"]), "graph_nodes_per_step": int(st["n_nodes"]),
            "roofline": {"bound": "hbm", "kernel": "decode GEMV family (mmvq_kernel<TYPE,1,MULTI>), the token's launch sequence timed alone",
                         "achieved": g["gbs"], "peak": peak, "unit": "GB/s", "frac": g["gbs"] / peak, "traffic": traffic, "traffic_source": traffic_src,
                         "peak_source": peak_src,
                         "alg_bytes_per_launch": g["alg_bytes_per_token"] / g["launches_per_token"], "avg_launch_us": g["avg_launch_us"],
                         "launches_per_step": g["launches_per_token"], "share_of_step": g["ms_per_token"] / (res_ms / steps)},
            "step_roofline": {"alg_bytes_per_step": wbytes + kvbytes, "achieved": (wbytes + kvbytes) / (res_ms / steps) / 1e6, "peak": peak, "unit": "GB/s",
                              "frac": (wbytes + kvbytes) / (res_ms / steps) / 1e6 / peak, "frac_of_8TBs_nominal": (wbytes + kvbytes) / (res_ms / steps) / 1e6 / 8000.0},
            "prefill": {"metric": "pp512_tokens_per_s", "value": PP_BATCH / (pp_best / 1e3), "ms": pp_best, "n_tokens": PP_BATCH,
                        "note": "same model, one 512-token batch at n_past=0 through b200_llama_decode (host sync timing, best of 3 after 1 warm-up)"},
            "clocks": clk, "setup_s": setup_s,
        }
        if tp70 is not None:
            line["tp_70b"] = tp70
        if world == 1 and not args.no_llamacpp:
            # the same metric through the REFERENCE's host code: unmodified llama.cpp + ggml_backend_sched drive libkcpp_b200.so
            # (Route 2 attach), host token ids in, host logits out, greedy; real 3968-token prompt in 512-token batches first
            try:
                j = run_harness(bench_gguf(shape), "b200", ["--n-prompt", N_PREFILLED, "--n-gen", min(steps, N_CTX - N_PREFILLED - 8), "--n-warm", 3, "--n-batch", PP_BATCH, "--n-ubatch", PP_BATCH])
                line["e2e_llamacpp"] = {"value": j["tg_tok_s"], "unit": UNIT, "pp_tokens_per_s": j["pp_tok_s"], "n_prompt": j["n_prompt"], "n_gen": j["n_gen"],
                                        "host": "reference llama.cpp (llama_decode, ggml_backend_sched) with the B200 backend attached by ggml_backend_register",
                                        "h2d_bytes_per_step": 4 + 4 + 4 * N_CTX * 32 + 4, "d2h_bytes_per_step": 4 * shape.n_vocab}
            except Exception as ex:
                line["e2e_llamacpp"] = {"value": None, "unit": UNIT, "error": f"{type(ex).__name__}: {ex}"[:300]}
        if world == 1 and not args.no_cpu:
            try:
                r = llamacpp_cpu_decode(shape, 16, 2)
                line["cpu_baseline"] = {"value": r["tok_s"], "unit": UNIT, "cores": r["cores"], "kind": "reference", "sample": r["sample"]}
            except Exception as ex:
                try:  # per-layer sample of the same compiled reference backend
                    sys.path.insert(0, str(ROOT / "tests"))
                    import cpu_baseline as B
                    r = B.time_decode(shape, N_CTX, budget_s=args.cpu_budget)
                    line["cpu_baseline"] = {"value": r["tok_s"], "unit": UNIT, "cores": r["cores"], "kind": "reference", "sample": r["sample"] + f" [llama.cpp harness unavailable: {ex}]"[:200]}
                except Exception as ex2:  # the checker library is prebuilt in oracle/_ref; its absence must not hide the GPU numbers
                    line["cpu_baseline"] = {"value": None, "unit": UNIT, "cores": 0, "kind": "reference", "sample": f"unavailable: {ex2}"}
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    return 0



# ------------------------------------------------------------------------------------------------ --design genesun
# Prefill and decode of the Genesun design at layer shapes of real model sizes (random bf16 weights), beside the llama decoder
# at equal width, depth and feed-forward size (Q4_K_M, the framework's flagship format).  Device time: the step's graph replayed
# with its inputs resident, CUDA events on the backend stream, an L2 flush (256 MB memset) before every timed replay.
DESIGN_SIZES = {
    # width, (attention: heads, dim, rot_dim, vdim, kv_rank, q_rank), (mLSTM: heads, dim, vdim), ff
    "w1024": (1024, (8, 64, 32, 64, 256, 384), (4, 128, 256), 2816),
    "w2048": (2048, (16, 128, 64, 128, 512, 768), (4, 256, 512), 5632),
    "w4096": (4096, (32, 128, 64, 128, 512, 1536), (8, 256, 512), 11008),
}
DESIGN_LAYERS, DESIGN_VOCAB, DESIGN_CTX, DESIGN_PP = 8, 32000, 1024, 512


def genesun_config(size: str) -> dict:
    import math
    W, (h, d, r, v, kr, qr), (mh, md, mv), ff = DESIGN_SIZES[size]
    rot = {"base": 10000.0, "dims": r, "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}
    layers = []
    for il in range(DESIGN_LAYERS):
        k = il % 4
        if k in (0, 3):
            layers.append({"type": "mlstm", "mixer": {"heads": mh, "dim": md, "vdim": mv, "gate_cap": 15.0}, "mlp": None})
        else:
            mx = {"heads": h, "dim": d, "rot_dim": r, "vdim": v, "kv_rank": kr, "q_rank": qr, "scale": 1.0 / math.sqrt(d + r), "rot": rot}
            if k == 2:
                mx["kv_from"] = il - 1
            layers.append({"type": "latent_attention", "mixer": mx, "mlp": {"kind": "dense", "ff": ff}})
    return {"architecture": "Genesun", "width": W, "vocab": DESIGN_VOCAB, "norm": {"eps": 1e-6}, "layers": layers}


def genesun_tensor_shapes(cfg: dict) -> dict:
    W, V = cfg["width"], cfg["vocab"]
    t = {"embed": (V, W), "head": (V, W), "final.norm": (W,)}
    for i, L in enumerate(cfg["layers"]):
        p, mx = f"l{i}.", L["mixer"]
        H, D, Vd = mx["heads"], mx["dim"], mx["vdim"]
        t.update({p + "norm1": (W,), p + "norm1b": (W,), p + "rg1": (W, W), p + "rg1.b": (W,), p + "dwa": (i + 2,)})
        if L["type"] == "mlstm":
            t.update({p + "mix.q": (H * D, W), p + "mix.k": (H * D, W), p + "mix.v": (H * Vd, W), p + "mix.g": (H * Vd, W), p + "mix.o": (W, H * Vd),
                      p + "mix.norm": (H * Vd,), p + "mix.i": (H, W), p + "mix.i.b": (H,), p + "mix.f": (H, W), p + "mix.f.b": (H,)})
        else:
            R, KR, QR = mx["rot_dim"], mx["kv_rank"], mx["q_rank"]
            t.update({p + "mix.dq": (QR, W), p + "mix.dq.norm": (QR,), p + "mix.uq": (H * (D + R), QR), p + "mix.uk": (H * D, KR), p + "mix.uv": (H * Vd, KR),
                      p + "mix.sink": (H,), p + "mix.g": (H * Vd, W), p + "mix.o": (W, H * Vd)})
            if "kv_from" not in mx:
                t.update({p + "mix.dkv": (KR + R, W), p + "mix.dkv.norm": (KR,)})
        if L["mlp"]:
            ff = L["mlp"]["ff"]
            t.update({p + "norm2": (W,), p + "norm2b": (W,), p + "rg2": (W, W), p + "rg2.b": (W,), p + "mlp.up": (ff, W), p + "mlp.down": (W, ff), p + "mlp.act": (4,)})
    return t


def genesun_random_tensors(cfg: dict, seed: int = 1):
    """Random weights of the right shapes (one pool of N(0, 0.02) values cut into the matrices; vectors near their neutral value)."""
    rng = np.random.default_rng(seed)
    pool = (rng.standard_normal(1 << 24, dtype=np.float32) * 0.02)
    pool_bits = ((pool.view(np.uint32) + 0x8000) >> 16).astype(np.uint16)
    out, at = {}, 0
    for name, shape in genesun_tensor_shapes(cfg).items():
        n = int(np.prod(shape))
        if len(shape) == 2 and name != "embed":
            reps = -(-n // len(pool_bits))
            bits = np.roll(pool_bits, at)[:n] if reps == 1 else np.tile(pool_bits, reps)[:n]
            at = (at + 7919 * 13) % len(pool_bits)
            out[name] = ("BF16", shape, bits.view(np.uint8))
        elif name == "embed":
            out[name] = ("F32", shape, np.resize(pool * 50, n).view(np.uint8))
        else:
            leaf = name.split(".")[-1]
            v = np.full(n, 1.0, np.float32) if "norm" in leaf else np.zeros(n, np.float32)
            if leaf == "dwa":
                v[:] = 1.0 / n
            if leaf == "act":
                v[:] = [0.6, 0.3, 0.1, 0.0]
            if name.endswith("f.b"):
                v[:] = 3.0
            out[name] = ("F32", shape, v.view(np.uint8))
    return out


def genesun_step_cost(cfg: dict, n_tokens: int, n_seq: int, ctx: int) -> dict:
    """Algorithmic bytes (bf16 weights once, latent cache rows and recurrent state of the batch) and FLOPs of one step."""
    W, V = cfg["width"], cfg["vocab"]
    wparams = W * V  # head
    cache = state = attn_flop = 0
    for L in cfg["layers"]:
        mx = L["mixer"]
        H, D, Vd = mx["heads"], mx["dim"], mx["vdim"]
        wparams += W * W + (2 * W * L["mlp"]["ff"] + W * W if L["mlp"] else 0)
        if L["type"] == "mlstm":
            wparams += W * (2 * H * D + 2 * H * Vd + 2 * H) + W * H * Vd
            state += n_seq * H * D * Vd * 4 * 2
        else:
            R, KR, QR = mx["rot_dim"], mx["kv_rank"], mx["q_rank"]
            wparams += W * QR + QR * H * (D + R) + H * D * KR + H * Vd * KR + 2 * W * H * Vd + (W * (KR + R) if "kv_from" not in mx else 0)
            cache += n_seq * ctx * (KR + R) * 4
            attn_flop += 2 * n_tokens * H * (ctx if n_tokens == n_seq else ctx // 2) * (2 * KR + R)
    return {"weight_bytes": 2 * wparams, "cache_bytes": cache, "state_bytes": state, "flop": 2 * wparams * n_tokens + attn_flop}



# ------------------------------------------------------------------------------------------------ --design galirax
# The same measurement for the Galirax design (grouped-query attention with sinks / windows, lightning attention, routed gated
# experts), beside the llama decoder with mixtral-style experts at equal width, depth, heads and expert sizes (Q4_K_M).
GALIRAX_SIZES = {
    # width, (heads, kv_heads, dim, vdim), (experts, per token, ff, groups, kept groups), window
    "w1024": (1024, (8, 2, 128, 128), (8, 2, 1024, 4, 2), 512),
    "w2048": (2048, (16, 4, 128, 128), (8, 2, 2048, 4, 2), 512),
    "w4096": (4096, (32, 8, 128, 128), (8, 2, 2048, 4, 2), 512),
}


def galirax_config(size: str) -> dict:
    import math
    W, (h, g, d, v), (ne, top, ff, ng, nk), window = GALIRAX_SIZES[size]
    mlp = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": ne, "top": top, "groups": {"count": ng, "keep": nk}, "scale": 2.0}}
    rot = {"base": 500000.0, "dims": d, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}
    layers = []
    for il in range(DESIGN_LAYERS):
        k = il % 4
        if k == 2:
            layers.append({"type": "lightning", "mixer": {"heads": h, "dim": d, "vdim": v, "decay": [1.0 - 2.0 ** (-5 - 3 * i / h) for i in range(h)]}, "mlp": mlp})
        elif k == 0:
            layers.append({"type": "attention", "mixer": {"heads": h, "kv_heads": g, "dim": d, "vdim": v, "rot": rot, "scale": 1.0 / math.sqrt(d)}, "mlp": mlp})
        else:
            layers.append({"type": "attention_2", "mixer": {"heads": h, "kv_heads": g, "dim": d, "vdim": v, "rot": {"base": 10000.0, "dims": d // 2}, "scale": 1.0 / math.sqrt(d),
                                                            "mask": {"size": window, "keep_first": 4}}, "mlp": mlp})
    return {"architecture": "Galirax", "width": W, "vocab": DESIGN_VOCAB, "norm": {"eps": 1e-5}, "logit_softcap": 30.0, "layers": layers}


def galirax_tensor_shapes(cfg: dict) -> dict:
    W, V = cfg["width"], cfg["vocab"]
    t = {"embed": (V, W), "head": (V, W), "final.norm": (W,), "final.norm.b": (W,)}
    for i, L in enumerate(cfg["layers"]):
        p, mx = f"l{i}.", L["mixer"]
        H, D, Vd = mx["heads"], mx["dim"], mx["vdim"]
        t.update({p + "norm1": (W,), p + "norm1.b": (W,), p + "mix.o": (W, H * Vd)})
        if L["type"] == "lightning":
            t.update({p + "mix.q": (H * D, W), p + "mix.k": (H * D, W), p + "mix.v": (H * Vd, W), p + "mix.g": (H * Vd, W), p + "mix.norm": (H * Vd,)})
        else:
            G = mx["kv_heads"]
            t.update({p + "mix.q": (H * D, W), p + "mix.k": (G * D, W), p + "mix.v": (G * Vd, W), p + "mix.sink": (H,)})
            if L["type"] == "attention_2":
                t.update({p + "mix.q.b": (H * D,), p + "mix.k.b": (G * D,), p + "mix.v.b": (G * Vd,), p + "mix.q.norm": (H * D,), p + "mix.k.norm": (G * D,)})
        if L["mlp"]:
            E, F = L["mlp"]["router"]["experts"], L["mlp"]["expert"]["ff"]
            t.update({p + "mlp.router": (E, W), p + "mlp.correction": (E,)})
            for e in range(E):
                t.update({f"{p}mlp.e{e}.gate": (F, W), f"{p}mlp.e{e}.up": (F, W), f"{p}mlp.e{e}.down": (W, F)})
    return t


def galirax_step_cost(cfg: dict, n_tokens: int, n_seq: int, ctx: int) -> dict:
    """Algorithmic bytes (bf16 weights once -- of the experts those a batch of this size can reach --, the visible f32 cache rows and
    the recurrent state of the batch) and FLOPs of one step."""
    W, V = cfg["width"], cfg["vocab"]
    wparams = W * V  # head
    active = W * V   # parameters a token multiplies with
    cache = state = attn_flop = 0
    for L in cfg["layers"]:
        mx = L["mixer"]
        H, D, Vd = mx["heads"], mx["dim"], mx["vdim"]
        if L["type"] == "lightning":
            p = W * (2 * H * D + 2 * H * Vd) + W * H * Vd
            state += n_seq * H * D * Vd * 4 * 2
            attn_flop += 4 * n_tokens * H * D * Vd
        else:
            G = mx["kv_heads"]
            p = W * (H * D + G * D + G * Vd) + W * H * Vd
            win = (mx.get("mask") or {}).get("size", 0)
            vis = min(ctx, win) if win else ctx
            cache += n_seq * vis * G * (D + Vd) * 4
            attn_flop += 2 * n_tokens * H * (vis if n_tokens == n_seq or win else ctx // 2) * (D + Vd)
        wparams += p
        active += p
        if L["mlp"]:
            r, F = L["mlp"]["router"], L["mlp"]["expert"]["ff"]
            wparams += W * r["experts"] + 3 * W * F * min(r["experts"], n_tokens * r["top"])
            active += W * r["experts"] + 3 * W * F * r["top"]
    return {"weight_bytes": 2 * wparams, "cache_bytes": cache, "state_bytes": state, "flop": 2 * active * n_tokens + attn_flop}


# ------------------------------------------------------------------------------------------------ --design zevopel
# The same measurement for the Zevopel design (norms behind the sublayers, chunked grouped-query attention with per-head q / k norms,
# sinks and head gates, a gated gelu feed-forward in the odd layers and softmax-routed clamped experts in the even ones), beside the
# closest existing model of the framework: Galirax with plain attention layers and routed experts at equal width, depth, heads and
# expert size, through the same loader, cache and engine.
ZEVOPEL_CHUNK = 8192


def zevopel_config(size: str) -> dict:
    import math
    W, (h, g, d, v), (ne, top, ff, _ng, _nk), _window = GALIRAX_SIZES[size]
    rot = {"base": 500000.0, "dims": d // 2, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}
    mixer = {"heads": h, "kv_heads": g, "dim": d, "vdim": v, "rot": rot, "scale": 1.0 / math.sqrt(d), "mask": {"size": ZEVOPEL_CHUNK}}
    moe = {"kind": "moe", "expert": {"ff": ff, "limit": 7.0}, "router": {"experts": ne, "top": top}}
    dense = {"kind": "dense", "ff": top * ff}  # as many active parameters as the routed layers
    layers = [{"type": "attention", "mixer": mixer, "mlp": moe if il % 2 == 0 else dense} for il in range(DESIGN_LAYERS)]
    return {"architecture": "Zevopel", "width": W, "vocab": DESIGN_VOCAB, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0}, "residual_mult": 1.0, "layers": layers}


def zevopel_tensor_shapes(cfg: dict) -> dict:
    W, V = cfg["width"], cfg["vocab"]
    t = {"embed": (V, W), "head": (V, W), "final.norm": (W,)}
    for i, L in enumerate(cfg["layers"]):
        p, mx = f"l{i}.", L["mixer"]
        H, G, D, Vd = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
        t.update({p + "norm1": (W,), p + "norm2": (W,), p + "ls1": (W,), p + "ls2": (W,), p + "mix.q": (H * D, W), p + "mix.k": (G * D, W), p + "mix.v": (G * Vd, W),
                  p + "mix.g": (H, W), p + "mix.o": (W, H * Vd), p + "mix.q.norm": (D,), p + "mix.k.norm": (D,), p + "mix.sink": (H,)})
        if L["mlp"]["kind"] == "dense":
            F = L["mlp"]["ff"]
            t.update({p + "mlp.gate": (F, W), p + "mlp.up": (F, W), p + "mlp.down": (W, F)})
        else:
            E, F = L["mlp"]["router"]["experts"], L["mlp"]["expert"]["ff"]
            t[p + "mlp.router"] = (E, W)
            for e in range(E):
                t.update({f"{p}mlp.e{e}.gate": (F, W), f"{p}mlp.e{e}.up": (F, W), f"{p}mlp.e{e}.down": (W, F)})
    return t


def zevopel_random_tensors(cfg: dict):
    out = random_tensors(zevopel_tensor_shapes(cfg))
    for name, (dt, shape, raw) in list(out.items()):
        leaf = name.split(".")[-1]
        if leaf in ("ls1", "ls2"):  # the per-channel scales sit near one, the norm weights (stored as the distance from one) near zero
            out[name] = (dt, shape, np.full(int(np.prod(shape)), 1.0, np.float32).view(np.uint8))
        elif leaf in ("norm1", "norm2") or name == "final.norm":
            out[name] = (dt, shape, np.zeros(int(np.prod(shape)), np.float32).view(np.uint8))
    return out


def zevopel_step_cost(cfg: dict, n_tokens: int, n_seq: int, ctx: int) -> dict:
    """Algorithmic bytes (bf16 weights once -- of the experts those a batch of this size can reach --, the visible f32 cache rows of the
    batch) and FLOPs of one step."""
    W, V = cfg["width"], cfg["vocab"]
    wparams = active = W * V  # head
    cache = attn_flop = 0
    for L in cfg["layers"]:
        mx = L["mixer"]
        H, G, D, Vd = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
        p = W * (H * D + G * D + G * Vd + H) + W * H * Vd
        vis = min(ctx, (mx.get("mask") or {}).get("size", 0) or ctx)
        cache += n_seq * vis * G * (D + Vd) * 4
        attn_flop += 2 * n_tokens * H * (vis if n_tokens == n_seq else ctx // 2) * (D + Vd)
        wparams += p
        active += p
        if L["mlp"]["kind"] == "dense":
            wparams += 3 * W * L["mlp"]["ff"]
            active += 3 * W * L["mlp"]["ff"]
        else:
            r, F = L["mlp"]["router"], L["mlp"]["expert"]["ff"]
            wparams += W * r["experts"] + 3 * W * F * min(r["experts"], n_tokens * r["top"])
            active += W * r["experts"] + 3 * W * F * r["top"]
    return {"weight_bytes": 2 * wparams, "cache_bytes": cache, "state_bytes": 0, "flop": 2 * active * n_tokens + attn_flop}


def zevopel_beside_config(size: str) -> dict:
    """Galirax at equal width, depth, heads and expert size: plain attention layers (sink, no window), routed experts in every layer."""
    import math
    W, (h, g, d, v), (ne, top, ff, ng, nk), _window = GALIRAX_SIZES[size]
    mlp = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": ne, "top": top, "groups": {"count": ng, "keep": nk}, "scale": 2.0}}
    rot = {"base": 500000.0, "dims": d // 2, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}
    layers = [{"type": "attention", "mixer": {"heads": h, "kv_heads": g, "dim": d, "vdim": v, "rot": rot, "scale": 1.0 / math.sqrt(d)}, "mlp": mlp} for _ in range(DESIGN_LAYERS)]
    return {"architecture": "Galirax", "width": W, "vocab": DESIGN_VOCAB, "norm": {"eps": 1e-5}, "logit_softcap": 30.0, "layers": layers}


# ------------------------------------------------------------------------------------------------ --design medodra
# The same measurement for the Medodra design (layers alternating between sigmoid attention beside a minGRU and the gated delta rule,
# short convolutions on q / k / v, sigmoid-routed experts weighted on their input plus a gated shared expert, one looped stretch with
# its input projection), beside the closest existing model of the framework: Galirax with alternating attention and lightning (linear
# attention) layers and routed experts in every layer at equal width, depth, heads and expert size.
def medodra_config(size: str) -> dict:
    import math
    W, (h, g, d, v), (ne, top, ff, _ng, _nk), _window = GALIRAX_SIZES[size]
    mlp = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": ne, "top": top}, "shared": {"ff": ff}}
    left = {"heads": h, "kv_heads": g, "dim": d, "vdim": v, "conv": 4, "bias_max": 2048, "q_temp": {"coef": 0.25, "every": 1024}, "scale": 1.0 / math.sqrt(d)}
    par = {"type": "parallel", "mixer": {"left": left, "right": {"width": W}}, "mlp": mlp}
    delta = {"type": "delta", "mixer": {"heads": h, "kv_heads": g, "dim": d, "vdim": v, "conv": 4}, "mlp": mlp}
    return {"architecture": "Medodra", "width": W, "vocab": DESIGN_VOCAB, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0}, "residual_mult": 0.7,
            "loop": {"start": 2, "stop": 4, "times": 1}, "layers": [par if il % 2 == 0 else delta for il in range(DESIGN_LAYERS)]}


def medodra_random_tensors(cfg: dict):
    W, V = cfg["width"], cfg["vocab"]
    t = {"embed": (V, W), "head": (V, W), "final.norm": (W,), "loop.in": (W, 2 * W)}
    for i, L in enumerate(cfg["layers"]):
        p, mx = f"l{i}.", L["mixer"]
        t.update({p + "norm1": (W,), p + "norm2": (W,)})
        if L["type"] == "delta":
            H, G, D, Vd, taps = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"], mx["conv"]
            t.update({p + "mix.q": (G * D, W), p + "mix.k": (G * D, W), p + "mix.v": (H * Vd, W), p + "mix.q.conv": (G * D, taps), p + "mix.k.conv": (G * D, taps),
                      p + "mix.v.conv": (H * Vd, taps), p + "mix.b": (H, W), p + "mix.a": (H, W), p + "mix.g": (H * Vd, W), p + "mix.o": (W, H * Vd), p + "mix.A_log": (H,),
                      p + "mix.dt_bias": (H,), p + "mix.norm": (Vd,)})
        else:
            a, side = mx["left"], mx["right"]["width"]
            H, G, D, Vd, taps = a["heads"], a["kv_heads"], a["dim"], a["vdim"], a["conv"]
            for leaf, rows in (("q", H * D), ("k", G * D), ("v", G * Vd)):
                t.update({p + "mix.left." + leaf: (rows, W), p + "mix.left." + leaf + ".b": (rows,), p + "mix.left." + leaf + ".conv": (rows, taps)})
            t.update({p + "mix.left.rel": (32, H), p + "mix.left.pb": (H,), p + "mix.left.o": (W, H * Vd), p + "mix.left.o.b": (W,), p + "mix.right.z": (side, W),
                      p + "mix.right.z.b": (side,), p + "mix.right.x": (side, W), p + "mix.right.x.b": (side,), p + "mix.right.g": (side, W), p + "mix.right.o": (W, side),
                      p + "mix.left.out": (W,), p + "mix.right.out": (W,)})
        E, F, FS = L["mlp"]["router"]["experts"], L["mlp"]["expert"]["ff"], L["mlp"]["shared"]["ff"]
        t.update({p + "mlp.router": (E, W), p + "mlp.shared.gate": (FS, W), p + "mlp.shared.up": (FS, W), p + "mlp.shared.down": (W, FS), p + "mlp.shared.sg": (1, W)})
        for e in range(E):
            t.update({f"{p}mlp.e{e}.gate": (F, W), f"{p}mlp.e{e}.up": (F, W), f"{p}mlp.e{e}.down": (W, F)})
    out = random_tensors(t)
    for name, (dt, shape, raw) in list(out.items()):
        leaf = name.split(".")[-1]
        if leaf in ("norm1", "norm2") or name == "final.norm":  # stored as the distance from one
            out[name] = (dt, shape, np.zeros(int(np.prod(shape)), np.float32).view(np.uint8))
        elif leaf == "out":
            out[name] = (dt, shape, np.full(int(np.prod(shape)), 1.0, np.float32).view(np.uint8))
    return out


def medodra_step_cost(cfg: dict, n_tokens: int, n_seq: int, ctx: int) -> dict:
    """Algorithmic bytes (bf16 weights once -- of the experts those a batch of this size can reach --, the f32 cache rows and recurrent
    states of the batch) and FLOPs of one step."""
    W, V = cfg["width"], cfg["vocab"]
    wparams = active = W * V + 2 * W * W  # head, loop.in (the stretch runs once)
    cache = state = attn_flop = 0
    for L in cfg["layers"]:
        mx = L["mixer"]
        if L["type"] == "delta":
            H, G, D, Vd = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
            p = W * (2 * G * D + 2 * H * Vd + 2 * H) + W * H * Vd
            state += n_seq * H * D * Vd * 4 * 2
            attn_flop += 6 * n_tokens * H * D * Vd
        else:
            a, side = mx["left"], mx["right"]["width"]
            H, G, D, Vd = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            p = W * (H * D + G * D + G * Vd + 3 * side) + W * H * Vd + W * side
            cache += n_seq * ctx * G * (D + Vd) * 4
            attn_flop += 2 * n_tokens * H * (ctx if n_tokens == n_seq else ctx // 2) * (D + Vd)
        r, F, FS = L["mlp"]["router"], L["mlp"]["expert"]["ff"], L["mlp"]["shared"]["ff"]
        wparams += p + W * r["experts"] + 3 * W * F * min(r["experts"], n_tokens * r["top"]) + 3 * W * FS + W
        active += p + W * r["experts"] + 3 * W * F * r["top"] + 3 * W * FS + W
    return {"weight_bytes": 2 * wparams, "cache_bytes": cache, "state_bytes": state, "flop": 2 * active * n_tokens + attn_flop}


def medodra_beside_config(size: str) -> dict:
    """Galirax at equal width, depth, heads and expert size: attention (sink, no window) and lightning layers in turn, routed experts in every layer."""
    import math
    W, (h, g, d, v), (ne, top, ff, ng, nk), _window = GALIRAX_SIZES[size]
    mlp = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": ne, "top": top, "groups": {"count": ng, "keep": nk}, "scale": 2.0}}
    rot = {"base": 500000.0, "dims": d // 2}
    att = {"type": "attention", "mixer": {"heads": h, "kv_heads": g, "dim": d, "vdim": v, "rot": rot, "scale": 1.0 / math.sqrt(d)}, "mlp": mlp}
    lin = {"type": "lightning", "mixer": {"heads": h, "dim": d, "vdim": v, "decay": [1.0 - 2.0 ** (-5 - 3 * i / h) for i in range(h)]}, "mlp": mlp}
    return {"architecture": "Galirax", "width": W, "vocab": DESIGN_VOCAB, "norm": {"eps": 1e-5}, "logit_softcap": 30.0, "layers": [att if il % 2 == 0 else lin for il in range(DESIGN_LAYERS)]}


def galirax_llama_shape(size: str):
    import koboldcpp_b200.llama as LL
    W, (h, g, d, v), (ne, top, ff, ng, nk), window = GALIRAX_SIZES[size]
    return LL.ModelShape(f"llama-moe-{size}", W, DESIGN_LAYERS, h, g, ff, DESIGN_VOCAB, "Q4_K_M", ne, top)


def genesun_llama_shape(size: str):
    import koboldcpp_b200.llama as LL
    W, _, _, ff = DESIGN_SIZES[size]
    return LL.ModelShape(f"llama-{size}", W, DESIGN_LAYERS, W // 128, W // 128, (ff + 255) // 256 * 256, DESIGN_VOCAB, "Q4_K_M")


def random_tensors(shapes: dict, seed: int = 1):
    """Random weights of the right shapes (one pool of N(0, 0.02) values cut into the matrices; vectors near their neutral value)."""
    rng = np.random.default_rng(seed)
    pool = (rng.standard_normal(1 << 24, dtype=np.float32) * 0.02)
    pool_bits = ((pool.view(np.uint32) + 0x8000) >> 16).astype(np.uint16)
    out, at = {}, 0
    for name, shape in shapes.items():
        n = int(np.prod(shape))
        if len(shape) == 2 and name != "embed":
            reps = -(-n // len(pool_bits))
            bits = np.roll(pool_bits, at)[:n] if reps == 1 else np.tile(pool_bits, reps)[:n]
            at = (at + 7919 * 13) % len(pool_bits)
            out[name] = ("BF16", shape, bits.view(np.uint8))
        elif name == "embed":
            out[name] = ("F32", shape, np.resize(pool * 50, n).view(np.uint8))
        else:
            leaf = name.split(".")[-1]
            v = np.full(n, 1.0, np.float32) if leaf.startswith("norm") else np.zeros(n, np.float32)
            if leaf == "correction":
                v[:] = np.resize(pool[:4096] * 5, n)
            out[name] = ("F32", shape, v.view(np.uint8))
    return out


def design_table():
    from koboldcpp_b200 import galirax, genesun, medodra, zevopel
    return {
        "medodra": {"sizes": GALIRAX_SIZES, "config": medodra_config, "tensors": medodra_random_tensors, "cost": medodra_step_cost, "build": medodra.build,
                    "beside_design": {"name": "galirax", "config": medodra_beside_config, "tensors": lambda cfg: random_tensors(galirax_tensor_shapes(cfg)),
                                      "cost": galirax_step_cost, "build": galirax.build},
                    "beside": "Galirax (attention with sinks and lightning layers in turn, routed experts in every layer), equal width / depth / heads / expert size, bf16"},
        "zevopel": {"sizes": GALIRAX_SIZES, "config": zevopel_config, "tensors": zevopel_random_tensors, "cost": zevopel_step_cost, "build": zevopel.build,
                    "beside_design": {"name": "galirax", "config": zevopel_beside_config, "tensors": lambda cfg: random_tensors(galirax_tensor_shapes(cfg)),
                                      "cost": galirax_step_cost, "build": galirax.build},
                    "beside": "Galirax (attention with sinks + routed experts in every layer), equal width / depth / heads / expert size, bf16"},
        "genesun": {"sizes": DESIGN_SIZES, "config": genesun_config, "tensors": lambda cfg: genesun_random_tensors(cfg), "cost": genesun_step_cost, "build": genesun.build,
                    "llama": genesun_llama_shape, "beside": "llama Q4_K_M, equal width / depth / ff"},
        "galirax": {"sizes": GALIRAX_SIZES, "config": galirax_config, "tensors": lambda cfg: random_tensors(galirax_tensor_shapes(cfg)), "cost": galirax_step_cost,
                    "build": galirax.build, "llama": galirax_llama_shape, "beside": "llama with routed experts Q4_K_M, equal width / depth / heads / experts"},
    }

def design_leg(args) -> int:
    import koboldcpp_b200.llama as LL
    DS = design_table()[args.design]
    name = args.design
    from koboldcpp_b200.engine import Engine
    from koboldcpp_b200.lib import F16, check, lib
    L = lib()
    if L.b200_device_count() <= 0:
        print("bench.py: no CUDA device and the product has no CPU path", file=sys.stderr)
        return 2
    hbm_gbs, _ = peaks()
    try:
        tfl = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()).get("bf16_tflops", 1590.0)
    except Exception:
        tfl = 1590.0
    flush = C.c_void_p()
    check(L.b200_malloc(C.byref(flush), 256 << 20))
    e0, e1 = C.c_void_p(), C.c_void_p()
    check(L.b200_event_create(C.byref(e0))); check(L.b200_event_create(C.byref(e1)))

    def time_replay(model, stream, steps, warmup):
        for _ in range(warmup):
            model.replay()
        total = 0.0
        for _ in range(steps):
            check(L.b200_memset(flush, 0, 256 << 20, stream))
            check(L.b200_event_record(e0, stream))
            model.replay()
            check(L.b200_event_record(e1, stream))
            check(L.b200_stream_synchronize(stream))
            ms = C.c_float()
            check(L.b200_event_elapsed_ms(e0, e1, C.byref(ms)))
            total += ms.value
        return total / steps

    steps, warmup = max(3, min(args.steps, 20)), max(3, args.warmup)

    def measure_design(DS, name, cfg, row, prompt, rng):
        m = DS["build"](cfg, DS["tensors"](cfg), dtype="bfloat16", n_ctx=8 * DESIGN_CTX + 256, n_seq_max=8, max_batch=DESIGN_PP)
        eng = Engine(m)
        # prefill: one prompt of DESIGN_PP tokens
        t0 = time.time()
        eng.step([("p", prompt, [DESIGN_PP - 1])])
        e2e_first = time.time() - t0
        ms = time_replay(m, m.stream, steps, warmup)
        cost = DS["cost"](cfg, DESIGN_PP, 1, DESIGN_PP)
        row[f"{name}_prefill"] = {"tokens": DESIGN_PP, "ms": ms, "tok_s": DESIGN_PP / ms * 1e3, "tflops": cost["flop"] / ms / 1e9,
                                  "of_measured_bf16": cost["flop"] / ms / 1e9 / tfl, "launches": m.stats()["n_kernels"], "first_call_s": e2e_first}
        eng.finish("p")
        # decode: 1 and 8 sequences at DESIGN_CTX tokens of context each
        for nseq in (1, 8):
            ids = [f"d{nseq}_{i}" for i in range(nseq)]
            for rid in ids:
                for a in range(0, DESIGN_CTX, DESIGN_PP):
                    eng.step([(rid, rng.integers(0, DESIGN_VOCAB, DESIGN_PP).tolist(), [])])
            t0 = time.time()
            n_e2e = 8
            for _ in range(n_e2e):
                lg = eng.step([(rid, [5], [0]) for rid in ids])
            e2e_ms = (time.time() - t0) / n_e2e * 1e3
            ms = time_replay(m, m.stream, steps, warmup)
            cost = DS["cost"](cfg, nseq, nseq, DESIGN_CTX)
            byt = cost["weight_bytes"] + cost["cache_bytes"] + cost["state_bytes"]
            row[f"{name}_decode_b{nseq}"] = {"ms": ms, "tok_s": nseq / ms * 1e3, "e2e_ms": e2e_ms, "e2e_tok_s": nseq / e2e_ms * 1e3, "alg_bytes": byt, "gbs": byt / ms / 1e6,
                                              "of_measured_hbm": byt / ms / 1e6 / hbm_gbs, "launches": m.stats()["n_kernels"], "finite": bool(np.isfinite(lg).all())}
            for rid in ids:
                eng.finish(rid)
        m.close()

    rows = []
    sizes = [s for s in DS["sizes"] if not args.design_sizes or s in args.design_sizes.split(",")]
    for size in sizes:
        cfg = DS["config"](size)
        W = cfg["width"]
        row = {"size": size, "width": W, "layers": DESIGN_LAYERS, "ctx": DESIGN_CTX}
        rng = np.random.default_rng(0)
        prompt = rng.integers(0, DESIGN_VOCAB, DESIGN_PP).tolist()
        measure_design(DS, name, cfg, row, prompt, rng)
        if "beside_design" in DS:  # the closest existing design at equal size, through the same loader, cache and engine
            BD = DS["beside_design"]
            measure_design(BD, BD["name"], BD["config"](size), row, prompt, rng)
            rows.append(row)
            print(json.dumps({"design_size": row}), file=sys.stderr, flush=True)
            continue
        # the llama decoder at equal width, depth and feed-forward size
        shape = DS["llama"](size)
        lm = LL.LlamaModel(shape, DESIGN_CTX + 256, F16)
        lm.init_random(seed=3)
        lm.finalize(max_batch=DESIGN_PP)
        lm.kv_fill_random(DESIGN_CTX, seed=7)
        lm.decode(prompt, 0)
        ms = time_replay(lm, lm.stream, steps, warmup)
        kvw = W * shape.n_head_kv // shape.n_head
        lflop = 2 * DESIGN_PP * (shape.n_layer * (2 * W * W + 2 * W * kvw + 3 * W * shape.n_ff * max(1, shape.n_expert_used) + W * shape.n_expert) + W * DESIGN_VOCAB) + \
            4 * DESIGN_PP * (DESIGN_PP // 2) * W * shape.n_layer
        row["llama_prefill"] = {"tokens": DESIGN_PP, "ms": ms, "tok_s": DESIGN_PP / ms * 1e3, "tflops": lflop / ms / 1e9, "of_measured_bf16": lflop / ms / 1e9 / tfl,
                                "launches": lm.stats()["n_kernels"]}
        lm.kv_fill_random(DESIGN_CTX, seed=7)
        lm.decode([5], DESIGN_CTX)
        ms = time_replay(lm, lm.stream, steps, warmup)
        byt = LL.weight_bytes_per_token(shape) + LL.kv_bytes_per_token(shape, DESIGN_CTX + 256, F16)
        row["llama_decode_b1"] = {"ms": ms, "tok_s": 1e3 / ms, "alg_bytes": byt, "gbs": byt / ms / 1e6, "of_measured_hbm": byt / ms / 1e6 / hbm_gbs, "launches": lm.stats()["n_kernels"]}
        lm.close()
        rows.append(row)
        print(json.dumps({"design_size": row}), file=sys.stderr, flush=True)
    print(json.dumps({"design": name, "beside": DS["beside"], "dtype": "bf16", "data": "synthetic", "steps": steps, "warmup": warmup,
                      "timing": "CUDA events around the replayed step graph, 256 MB L2 flush before each", "sizes": rows}))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=125)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-llamacpp", action="store_true", help="skip the e2e_llamacpp leg (reference llama.cpp driving the B200 backend)")
    ap.add_argument("--cpu-budget", type=float, default=18.0)
    ap.add_argument("--no-tp70", action="store_true", default=bool(os.environ.get("B200_BENCH_NO_TP70")),
                    help="skip the auxiliary 70B tensor-parallel leg (BASELINE.json configs[4])")
    ap.add_argument("--design", default="", choices=["", "genesun", "galirax", "zevopel", "medodra"],
                    help="instead of the default workload: prefill / decode of this design at real layer shapes beside the closest existing model at equal size")
    ap.add_argument("--design-sizes", default="", help="comma-separated subset of the sizes of the design (genesun: " + ",".join(DESIGN_SIZES) + "; the others: " + ",".join(GALIRAX_SIZES) + ")")
    args = ap.parse_args()
    if args.design:
        return design_leg(args)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        return reference_arm(args, rank)
    return product_arm(args, rank, world, local_rank)


if __name__ == "__main__":
    sys.exit(main())
