#!/usr/bin/env python
"""Benchmark of the quantized-matmul hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload (the configuration the headline metric is quoted on): GGUF Q4_K prefill dequant-GEMM,
activations M = 512 tokens x K = 4096 (bf16, N(0,1)), weights N = 14336 x K = 4096 in Q4_K super-blocks
(f16 d and dmin ~ |N(0, 0.01)|, uniform 6-bit scales / mins, uniform 4-bit quants), f32 output.
One step = one pass of that matmul over the 512-token batch. Seeded synthetic data.

On N > 1 GPUs the weight rows are sharded (tensor parallel, N / world rows per rank): every rank multiplies the same
activations by its shard and the ranks then all-gather the output over NVLink (NCCL), both inside the timed step; total
work is fixed, so scaling is "strong". Before timing, every rank checks that its shard's output equals the same rows of
the unsharded product bit for bit (`config.parity`). Timing is on the device (CUDA events on the launching stream,
barrier + synchronize on both sides, max over ranks); the block of --steps steps is repeated until the timed region
holds at least 0.3 s of device time (`repeats`), and `ms_per_step` is the mean over all of them.

Prints ONE JSON line on rank 0. `value` is whole-job TFLOP/s with inputs resident in HBM; `e2e` is the
same metric through the host-buffer call of the C ABI (b2_matmul: pinned f32 x in, f32 y out, both
copies inside the timed region); `roofline` is the tensor-core GEMM kernel alone against the measured
bf16 peak; `cpu_baseline` is the CPU oracle's restatement of the reference's AVX2 prefill path on
the box's host cores. `--impl reference` times only that CPU path, on the same workload.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

M_TOK, K_IN, N_OUT = 512, 4096, 14336
FLOP_PER_STEP = 2.0 * M_TOK * K_IN * N_OUT
WORKLOAD = "gguf_q4_k_prefill_gemm M=512 K=4096 N=14336 (bf16 activations, f32 output)"
METRIC = "prefill dequant-GEMM throughput (Q4_K, M=512 K=4096 N=14336)"
L2_BYTES = 126 * 1024 * 1024

def profiled_traffic(name: str):
    """dram__bytes_read.sum + dram__bytes_write.sum per launch of a kernel, read from the ncu summary committed under
    profiles/ (lines `dram__bytes_read.sum: N` / `dram__bytes_write.sum: N`, and `captured at: <commit>`); None when the
    file or the fields are missing."""
    import re

    f = ROOT / "profiles" / name
    if not f.exists():
        return None, None
    text = f.read_text()
    r = re.search(r"dram__bytes_read\.sum:\s*([0-9][0-9,_]*)", text)
    w = re.search(r"dram__bytes_write\.sum:\s*([0-9][0-9,_]*)", text)
    c = re.search(r"captured at:\s*(\S+)", text)
    if not r or not w:
        return None, None
    num = lambda m: int(m.group(1).replace(",", "").replace("_", ""))
    return num(r) + num(w), (c.group(1) if c else None)


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d.get("bf16_tflops_sustained"),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.index)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm = [float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        reasons = set()
        for r in self.rows:
            if len(r) >= 9:
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def cpu_prefill_tflops(threads: int, steps: int, warmup: int):
    """The reference's CPU prefill path (dequantize 8 rows + f32 FMA tiles, src/kernels.rs:1998-2038)
    as restated by the oracle, on the full workload, all host threads."""
    from oracle import oracle as O
    from oxinfer_b200 import synth

    ref = synth.q4_k(N_OUT, K_IN, 1)
    m = O.Matrix.gguf(O.Q4_K, ref.data, N_OUT, K_IN)
    x = synth.activations(M_TOK, K_IN, 2)
    for _ in range(warmup):
        m.matmul_cpu(x, threads)
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        m.matmul_cpu(x, threads)
        times.append(time.perf_counter() - t0)
    return times


def base_config(world: int) -> dict:
    """The `config` both arms print (same keys, same values)."""
    return {"workload": WORKLOAD,
            "parallelism": (f"tp{world}: weight rows sharded, every rank ends each step with the whole y (gathered by the GEMM epilogue's peer stores "
                            "over NVLink, or by an NCCL all-gather where that path is declined)") if world > 1 else "single GPU",
            "l2": "inputs larger than L2: rotating over weight copies of more than twice the L2 size"}


def run_reference(args, rank):
    if rank != 0:
        return
    from oracle import oracle as O

    threads = O.cpu_threads()
    steps, warm = max(1, args.steps), max(1, args.warmup)
    times = cpu_prefill_tflops(threads, steps, warm)
    ms = 1e3 * sum(times) / len(times)
    v = FLOP_PER_STEP / (ms * 1e-3) / 1e12
    line = {
        "impl": "reference", "metric": METRIC, "value": v, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": steps, "warmup": warm,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": base_config(args.gpus),
        "path": "CPU: dequantize 8 rows + 8x8 f32 FMA tiles (oracle port of the reference's AVX2 prefill path, src/kernels.rs:1998-2038)",
        "cpu_baseline": {"value": v, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": "full workload (512 tokens x 14336 rows) per step"},
        "e2e": {"value": v, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(json.dumps(line))


def gemv_extras(be, torch, peaks, steps, only=None, use_graph=True):
    """Achieved HBM GB/s of the batch-1 dequant-GEMV kernels (algorithmic bytes / CUDA-event time),
    rotating over weight copies larger than L2."""
    from oxinfer_b200 import synth

    out = {}
    cases = [("mlx4_4096x4096", "mlx4", 4096, 4096), ("q4_k_14336x4096", "q4_k", 14336, 4096), ("q6_k_32064x4096", "q6_k", 32064, 4096),
             ("f8_e4m3_7168x12288", "f8_e4m3", 7168, 12288)]
    for name, fmt, n_out, n_in in [c for c in cases if not only or only in c[0]]:
        ref = synth.make(fmt, n_out, n_in, 5)
        dev0 = be.upload(ref, n_out, n_in)
        wbytes = dev0.bytes()
        copies = max(2, min(48, -(-2 * L2_BYTES // wbytes)))
        devs = [dev0] + [be.upload(ref, n_out, n_in) for _ in range(copies - 1)]
        x = torch.randn(n_in, device="cuda", dtype=torch.float32)
        y = torch.empty(n_out, device="cuda", dtype=torch.float32)
        for i in range(3):
            be.matvec_dev(devs[i % copies], x, y)
        torch.cuda.synchronize()
        # One GEMV is a few microseconds, less than a host launch: time a CUDA graph of n back-to-back
        # GEMVs (each with its activation-plane kernel) over the rotating weight copies.
        n = max(steps, 2 * copies)
        graph, timing = torch.cuda.CUDAGraph(), "cuda graph"
        main_stream = torch.cuda.current_stream().cuda_stream
        try:
            if not use_graph:
                raise RuntimeError("graph timing switched off")
            with torch.cuda.graph(graph):
                be.set_stream(torch.cuda.current_stream().cuda_stream)
                for i in range(n):
                    be.matvec_dev(devs[i % copies], x, y)
            be.set_stream(main_stream)
            graph.replay()
            torch.cuda.synchronize()
        except Exception as e:
            be.set_stream(main_stream)
            graph, timing = None, f"host-launched ({type(e).__name__})"
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        reps = 5 if graph is not None else 1
        ev[0].record()
        for _ in range(reps):
            if graph is not None:
                graph.replay()
            else:
                for i in range(n):
                    be.matvec_dev(devs[i % copies], x, y)
        ev[1].record()
        torch.cuda.synchronize()
        us = ev[0].elapsed_time(ev[1]) * 1e3 / (n * reps)
        algo = wbytes + 4 * n_in + 4 * n_out
        out[name] = {"us_per_gemv": us, "bytes": algo, "gbs": algo / us / 1e3, "frac_of_hbm_peak": algo / us / 1e3 / peaks["hbm_gbs"],
                     "launches_per_gemv": 1 if fmt == "f8_e4m3" else 2, "timing": timing}
        traffic, commit = profiled_traffic(f"gemv_{name}.txt")
        out[name]["roofline"] = {"kernel": "gemv_f8_mma_kernel" if fmt == "f8_e4m3" else "xplanes_kernel + gemv_kernel (one matrix-vector product)",
                                 "bound": "hbm", "achieved": algo / us / 1e3, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                 "frac": algo / us / 1e3 / peaks["hbm_gbs"], "frac_of_nominal_8000": algo / us / 1e3 / 8000.0, "traffic": traffic,
                                 "traffic_unit": f"bytes per product, from profiles/gemv_{name}.txt" + (f" captured at {commit}" if commit else ""),
                                 "bytes_per_launch": algo, "peak_source": f"copy bandwidth, {peaks['source']}"}
        if name.startswith("mlx4") or name.startswith("q4_k"):
            # the same product through the host-buffer call (Backend::matvec_rows): pinned x in, y out, synchronous
            xh = torch.randn((1, n_in), dtype=torch.float32).pin_memory()
            yh = torch.empty((1, n_out), dtype=torch.float32).pin_memory()
            import oxinfer_b200 as ob

            for i in range(3):
                assert be.matvec_rows(xh.numpy(), [ob.RowsJob(devs[i % copies], yh.numpy())])
            torch.cuda.synchronize()
            ev[0].record()
            for i in range(n):
                be.matvec_rows(xh.numpy(), [ob.RowsJob(devs[i % copies], yh.numpy())])
            ev[1].record()
            torch.cuda.synchronize()
            us_e = ev[0].elapsed_time(ev[1]) * 1e3 / n
            out[name]["e2e"] = {"value": algo / us_e / 1e3, "unit": "GB/s", "us_per_gemv": us_e, "h2d_bytes_per_step": 4 * n_in, "d2h_bytes_per_step": 4 * n_out,
                                "call": "b2_matvec_rows (Backend::matvec_rows): host f32 x in, f32 y out, synchronous"}
            # the reference's CPU decode path for this product (int8 activations, oracle port), all host threads
            try:
                from oracle import oracle as O

                m = O.matrix_of(ref, n_out, n_in)
                xc = xh.numpy()
                m.matmul_cpu(xc)
                reps_c, t0 = 0, time.perf_counter()
                while time.perf_counter() - t0 < 1.0:
                    m.matmul_cpu(xc)
                    reps_c += 1
                us_c = (time.perf_counter() - t0) / reps_c * 1e6
                out[name]["cpu_baseline"] = {"value": algo / us_c / 1e3, "unit": "GB/s", "cores": O.cpu_threads(), "kind": "port",
                                             "sample": f"{reps_c} products in 1 s (one matrix: it stays in the CPU's cache, which favours the CPU)",
                                             "path": O.decode_kernel_name()}
            except Exception as e:
                out[name]["cpu_baseline_error"] = str(e)
        # The GEMV kernel alone, over planes prepared once (what a decode plan sees when one vector feeds
        # several products): a second graph with n GEMV launches and no plane kernels.
        if use_graph and fmt != "f8_e4m3":
            try:
                be.prepare_x_dev(x)
                g2 = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g2):
                    be.set_stream(torch.cuda.current_stream().cuda_stream)
                    for i in range(n):
                        be.matvec_prepared_dev(devs[i % copies], x, y)
                be.set_stream(main_stream)
                g2.replay()
                torch.cuda.synchronize()
                ev[0].record()
                for _ in range(5):
                    g2.replay()
                ev[1].record()
                torch.cuda.synchronize()
                us2 = ev[0].elapsed_time(ev[1]) * 1e3 / (n * 5)
                out[name].update({"us_kernel_only": us2, "gbs_kernel_only": algo / us2 / 1e3,
                                  "frac_kernel_only": algo / us2 / 1e3 / peaks["hbm_gbs"]})
                # the same as a dependent-launch chain (how a decode step queues its products): every kernel may start while
                # the one ahead drains, and the 4-bit kernels fetch their first weights before they wait for it
                be.set_chained(True)
                g3 = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g3):
                    be.set_stream(torch.cuda.current_stream().cuda_stream)
                    for i in range(n):
                        be.matvec_prepared_dev(devs[i % copies], x, y)
                be.set_stream(main_stream)
                be.set_chained(False)
                g3.replay()
                torch.cuda.synchronize()
                ev[0].record()
                for _ in range(5):
                    g3.replay()
                ev[1].record()
                torch.cuda.synchronize()
                us3 = ev[0].elapsed_time(ev[1]) * 1e3 / (n * 5)
                out[name].update({"us_chained": us3, "gbs_chained": algo / us3 / 1e3, "frac_chained": algo / us3 / 1e3 / peaks["hbm_gbs"]})
            except Exception as e:
                be.set_stream(main_stream)
                be.set_chained(False)
                out[name]["kernel_only_error"] = str(e)
        if fmt == "mlx4":
            # the reference's own CUDA kernel for this product (dmv_q4a, compiled for sm_100a into oracle/_ref where the
            # reference's tree was present at build time), host-launched back to back on the same matrix
            try:
                from oracle import oracle as O

                L = O.ref_cuda()
                if L is not None:
                    m = O.Matrix.from_mlx_q4(ref.w.reshape(-1), ref.scales.reshape(-1), ref.biases.reshape(-1), n_out, n_in, ref.group)
                    ms = O.ref_dmv_q4a(L, m, x, y, iters=200, stream=torch.cuda.current_stream().cuda_stream)
                    out[name]["reference_cuda_kernel"] = {"kernel": "dmv_q4a (src/cuda_decode.cu), 4 warps x 4 rows per block", "us": ms * 1e3,
                                                          "note": "one matrix, 200 launches back to back: its 9.5 MB stay in L2, which favours it"}
            except Exception as e:
                out[name]["reference_cuda_kernel_error"] = str(e)
        for d in devs:
            d.free()
    if not only or "other" in only:
        out["other_formats"] = other_format_gemv(be, torch, peaks, steps)
    return out


def other_format_gemv(be, torch, peaks, steps):
    """The generic (untuned) matrix-vector kernel of the other GGUF block formats at 8192 x 4096: algorithmic bytes / CUDA-event
    time over rotating weight copies larger than L2, host-launched back to back."""
    from oxinfer_b200 import synth

    out = {}
    n_out, n_in = 8192, 4096
    x = torch.randn(n_in, device="cuda", dtype=torch.float32)
    y = torch.empty(n_out, device="cuda", dtype=torch.float32)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    for kind, name in synth.OTHER_NAMES.items():
        ref = synth.other_blocks(kind, n_out, n_in, 9)
        dev0 = be.upload(ref, n_out, n_in)
        if dev0 is None:
            out[name] = {"declined": be.last_declined}
            continue
        wbytes = dev0.bytes()
        copies = max(2, min(48, -(-2 * L2_BYTES // wbytes)))
        devs = [dev0] + [be.upload(ref, n_out, n_in) for _ in range(copies - 1)]
        n = max(steps, 2 * copies)
        for i in range(3):
            be.matvec_dev(devs[i % copies], x, y)
        torch.cuda.synchronize()
        ev[0].record()
        for i in range(n):
            be.matvec_dev(devs[i % copies], x, y)
        ev[1].record()
        torch.cuda.synchronize()
        us = ev[0].elapsed_time(ev[1]) * 1e3 / n
        algo = wbytes + 4 * n_in + 4 * n_out
        out[name] = {"us_per_gemv": us, "bytes": algo, "gbs": algo / us / 1e3, "frac_of_hbm_peak": algo / us / 1e3 / peaks["hbm_gbs"],
                     "kernel": "gemv_other_kernel", "shape": f"{n_out}x{n_in}"}
        for d in devs:
            d.free()
    return out


def ref_cuda_extras(be, torch):
    """The reference's own CUDA kernels (compiled for sm_100a into oracle/_ref where the reference's tree was present at
    build time) beside this repository's on the same device: the prefill product at config 1's shape on an MLX 4-bit
    matrix (the format gemm_q4a takes), and the reference's decode attention at config 2's shape."""
    import numpy as np

    import oxinfer_b200 as ob
    from oracle import oracle as O
    from oxinfer_b200 import synth

    L = O.ref_cuda()
    if L is None:
        return {"unavailable": "oracle/_ref/libref_cuda.so was not built"}
    out = {}
    ref = synth.mlx4(N_OUT, K_IN, 77)
    m = O.Matrix.from_mlx_q4(ref.w.reshape(-1), ref.scales.reshape(-1), ref.biases.reshape(-1), N_OUT, K_IN, ref.group)
    dev = be.upload(ref, N_OUT, K_IN)
    x = torch.from_numpy(synth.activations(M_TOK, K_IN, 78)).cuda()
    y_ref = torch.empty((M_TOK, N_OUT), device="cuda")
    ms_ref = O.ref_gemm_q4a(L, m, x, y_ref, iters=5)
    x16 = x.to(torch.float16)
    y = torch.empty((M_TOK, N_OUT), device="cuda")
    for _ in range(3):
        assert be.matmul_dev(dev, x16, y)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(20):
        be.matmul_dev(dev, x16, y)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / 20
    scale = float(y_ref.abs().max())
    out["prefill_mlx4_512x4096x14336"] = {
        "reference_kernel": "gemm_q4a (KERNEL_SRC of src/cuda.rs): 64 x 64 tiles, f32 FMA", "reference_us": ms_ref * 1e3,
        "reference_tflops": FLOP_PER_STEP / (ms_ref * 1e-3) / 1e12, "this_us": ms * 1e3, "this_tflops": FLOP_PER_STEP / (ms * 1e-3) / 1e12,
        "max_abs_difference_over_max": float((y - y_ref).abs().max()) / scale,
        "note": "one 29 MB matrix on both sides, launches back to back (weights stay in L2 for both)"}
    dev.free()
    nh, nkv, hd, pos = 32, 8, 128, 2048
    rng = np.random.default_rng(5)
    kc = torch.from_numpy(rng.standard_normal((pos + 1, nkv * hd)).astype(np.float32)).cuda()
    vc = torch.from_numpy(rng.standard_normal((pos + 1, nkv * hd)).astype(np.float32)).cuda()
    q = torch.from_numpy(rng.standard_normal(nh * hd).astype(np.float32)).cuda()
    o = torch.empty(nh * hd, device="cuda")
    sp = torch.tensor([pos, pos, 1, 0], dtype=torch.int32, device="cuda")
    ms_att = O.ref_attend(L, q, kc, vc, o, sp, nh, nkv, hd, hd ** -0.5, iters=100)
    out["decode_attention_32h_8kv_128_ctx2048"] = {
        "reference_kernels": "dattn_4_4 + dattn_combine (src/cuda_decode.cu)", "reference_us": ms_att * 1e3,
        "note": "this repository's attend kernel at the same shape: see the decode step's launch list under profiles/"}
    return out


def moe_extras(be, torch, peaks):
    """Config 3: the routed-expert layer (128 experts, top-8, hidden 2048, expert intermediate 768, MLX 4-bit g64) at token
    batches 1 / 64 / 512 / 4096, x and y on the device, routes on the host as in Backend::moe. Router logits N(0,1) plus a
    per-expert bias N(0,1) (skewed load), softmax over the 8 chosen. Eight distinct random experts are uploaded 16 times each
    (generation time only; every expert has its own device memory)."""
    import numpy as np

    from oxinfer_b200 import synth

    E, K, H, I = 128, 8, 2048, 768
    protos = [(synth.mlx4(2 * I, H, 900 + i), synth.mlx4(H, I, 950 + i)) for i in range(8)]
    gu = [be.upload(protos[e % 8][0], 2 * I, H) for e in range(E)]
    dn = [be.upload(protos[e % 8][1], H, I) for e in range(E)]
    moe = be.upload_moe(gu, dn, H, I)
    if moe is None:
        raise RuntimeError("upload_moe declined: " + be.last_declined)
    wbytes = sum(d.bytes() for d in gu) + sum(d.bytes() for d in dn)
    for d in gu + dn:
        d.free()
    rng = np.random.default_rng(3)
    bias = rng.standard_normal(E).astype(np.float32)
    out = {}
    for t in (1, 64, 512, 4096):
        logits = rng.standard_normal((t, E)).astype(np.float32) + bias
        ids = np.argsort(-logits, axis=1, kind="stable")[:, :K].astype(np.int32)
        top = np.take_along_axis(logits, ids, axis=1)
        w = np.exp(top - top[:, :1])
        w = (w / w.sum(axis=1, keepdims=True)).astype(np.float32)
        x = torch.randn((t, H), device="cuda", dtype=torch.float32)
        y = torch.zeros((t, H), device="cuda", dtype=torch.float32)
        for _ in range(2):
            be.moe_dev(x, ids, w, moe, y)
        torch.cuda.synchronize()
        be.check_status()
        n = 5
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            be.moe_dev(x, ids, w, moe, y)
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / n
        flop = 6.0 * t * K * H * I
        touched = len(np.unique(ids)) / E * wbytes
        out[f"t{t}"] = {"us": us, "tflops": flop / us / 1e6, "experts_touched": int(len(np.unique(ids))), "weight_gbs": touched / us / 1e3,
                        "frac_of_hbm_peak": touched / us / 1e3 / peaks["hbm_gbs"], "frac_of_bf16_peak": flop / us / 1e6 / peaks["bf16_tflops"]}
    out["note"] = "b2_moe_dev per call: host segment building + gather, grouped tensor-core GEMM (gate_up), SiLU, grouped GEMM (down), combine"
    # The reference's own CUDA kernels for the same layer on the same device (moe_gather, a gemm_q4a per touched expert and
    # projection, moe_act, moe_combine: the launch sequence of CudaBackend::moe_run, src/cuda.rs:798-966), device time only
    # (its host-side segment building and its three PCIe copies per call are left out, which favours it).
    try:
        from oracle import oracle as O

        L = O.ref_cuda()
        if L is None:
            out["reference_cuda"] = {"unavailable": "oracle/_ref/libref_cuda.so was not built"}
        else:
            pm = [(O.matrix_of(g, 2 * I, H), O.matrix_of(d, H, I)) for g, d in protos]
            rm = O.RefMoe([pm[e % 8][0] for e in range(E)], [pm[e % 8][1] for e in range(E)], H, I)
            refs = {}
            rng = np.random.default_rng(3)
            bias = rng.standard_normal(E).astype(np.float32)
            for t in (1, 64, 512, 4096):
                logits = rng.standard_normal((t, E)).astype(np.float32) + bias
                ids = np.argsort(-logits, axis=1, kind="stable")[:, :K].astype(np.int32)
                top = np.take_along_axis(logits, ids, axis=1)
                w = np.exp(top - top[:, :1])
                w = (w / w.sum(axis=1, keepdims=True)).astype(np.float32)
                x = torch.randn((t, H), device="cuda", dtype=torch.float32)
                y_ref = torch.zeros((t, H), device="cuda", dtype=torch.float32)
                O.ref_moe_q4a(L, rm, x, ids, w, y_ref, iters=0)
                y = torch.zeros((t, H), device="cuda", dtype=torch.float32)
                be.moe_dev(x, ids, w, moe, y)
                torch.cuda.synchronize()
                diff = float((y - y_ref).abs().max() / y_ref.abs().max())
                scratch = torch.zeros((t, H), device="cuda", dtype=torch.float32)
                ms = O.ref_moe_q4a(L, rm, x, ids, w, scratch, iters=3 if t >= 512 else 10)
                refs[f"t{t}"] = {"reference_us": ms * 1e3, "this_us": out[f"t{t}"]["us"], "speedup": ms * 1e3 / out[f"t{t}"]["us"],
                                 "max_abs_difference_over_max": diff}
            refs["note"] = "same routing distribution and experts; the reference sequence is 2 + 2 x (touched experts) + 1 launches per layer"
            out["reference_cuda"] = refs
    except Exception as e:
        out["reference_cuda_error"] = str(e)
    return out


def moe_ep_extras(be, torch, dist, rank, world):
    """Config 3 expert-parallel across the ranks (one process per GPU): 128 experts in equal contiguous shares, the token batch
    split evenly over the ranks, every (token, route) pair sent to the rank that owns its expert and back (b2_moe_ep: NCCL
    all-gather of the counts, grouped send / receive of the rows, local experts, ordered combine). Times one layer call at
    512 and 4096 tokens (whole batch over all ranks), slowest rank; before timing, rank 0's rows are checked against the
    one-GPU layer over all experts (bit for bit)."""
    import numpy as np

    import oxinfer_b200 as ob
    from oxinfer_b200 import synth

    E, K, H, I = 128, 8, 2048, 768
    assert E % world == 0
    if not getattr(be, "comm_ready", False):
        box = [ob.Backend.comm_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        be.comm_init(world, rank, box[0])
        be.comm_ready = True
    protos = [(synth.mlx4(2 * I, H, 900 + i), synth.mlx4(H, I, 950 + i)) for i in range(8)]
    pe = E // world
    gu = [be.upload(protos[e % 8][0], 2 * I, H) for e in range(rank * pe, (rank + 1) * pe)]
    dn = [be.upload(protos[e % 8][1], H, I) for e in range(rank * pe, (rank + 1) * pe)]
    local = be.upload_moe(gu, dn, H, I)
    for d in gu + dn:
        d.free()
    full = None
    if rank == 0:
        agu = [be.upload(protos[e % 8][0], 2 * I, H) for e in range(E)]
        adn = [be.upload(protos[e % 8][1], H, I) for e in range(E)]
        full = be.upload_moe(agu, adn, H, I)
        for d in agu + adn:
            d.free()
    out = {}
    rng = np.random.default_rng(3)
    bias = rng.standard_normal(E).astype(np.float32)
    for t in (512, 4096):
        logits = rng.standard_normal((t, E)).astype(np.float32) + bias
        ids = np.argsort(-logits, axis=1, kind="stable")[:, :K].astype(np.int32)
        top = np.take_along_axis(logits, ids, axis=1)
        w = np.exp(top - top[:, :1])
        w = (w / w.sum(axis=1, keepdims=True)).astype(np.float32)
        xs = synth.activations(t, H, 77 + t)
        share = t // world
        t0, t1 = rank * share, (rank + 1) * share
        x = torch.from_numpy(xs[t0:t1]).cuda()
        y = torch.zeros((share, H), device="cuda")
        be.moe_ep(x, ids[t0:t1], w[t0:t1], local, E, y)
        torch.cuda.synchronize()
        same = 1
        if rank == 0:
            want = torch.zeros((share, H), device="cuda")
            be.moe_dev(x, ids[t0:t1], w[t0:t1], full, want)
            torch.cuda.synchronize()
            same = int(torch.equal(want.view(torch.int32), y.view(torch.int32)))
        flag = torch.tensor([same], device="cuda", dtype=torch.int32)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        n = 5
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            be.moe_ep(x, ids[t0:t1], w[t0:t1], local, E, y)
        e1.record()
        torch.cuda.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1) / n], device="cuda", dtype=torch.float64)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        us = float(ms.item()) * 1e3
        flop = 6.0 * t * K * H * I
        out[f"t{t}"] = {"us": us, "tflops": flop / us / 1e6, "tokens_per_rank": share,
                        "parity": "bit-identical to the one-GPU layer (rank 0's rows)" if int(flag.item()) == 1 else "MISMATCH"}
    out["note"] = (f"ep{world}: {pe} experts per rank; per call an all-gather of counts (one host read), two grouped send / receive exchanges of "
                   "f32 rows, the local grouped-expert kernels, the ordered combine")
    be.comm_free()
    return out


def fp8_extras(be, torch, peaks):
    """Config 4: FP8 e4m3 128x128-block-scaled weights N=28672 x K=12288, f16 activations on the device, M = 128 and 8192
    through the tensor-core GEMM (M = 1 is the f8 case of extra.gemv at another shape). FP8 keeps the reference's
    semantics: e4m3 weight times block scale against unquantized activations, f32 accumulation."""
    from oxinfer_b200 import synth

    n_out, n_in = 28672, 12288
    ref = synth.f8_e4m3(n_out, n_in, 1)
    dev = be.upload(ref, n_out, n_in)
    out = {}
    # M = 1: the matrix-vector product (one launch; the 352 MB matrix is larger than L2 by itself)
    x1 = torch.randn(n_in, device="cuda", dtype=torch.float32)
    y1 = torch.empty(n_out, device="cuda", dtype=torch.float32)
    for _ in range(3):
        be.matvec_dev(dev, x1, y1)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(20):
        be.matvec_dev(dev, x1, y1)
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / 20
    wb = n_out * n_in + (n_out // 128) * (n_in // 128) * 4
    out["m1"] = {"us": us, "weight_gbs": wb / us / 1e3, "frac_of_hbm_peak": wb / us / 1e3 / peaks["hbm_gbs"],
                 "kernel": "gemv_f8_mma_kernel (mma.sync m16n8k16, x as two f16 columns)", "timing": "host-launched, 20 back to back"}
    for t in (128, 8192):
        xd = torch.randn((t, n_in), device="cuda", dtype=torch.float16)
        y = torch.empty((t, n_out), device="cuda", dtype=torch.float32)
        for _ in range(2):
            be.matmul_dev(dev, xd, y)
        torch.cuda.synchronize()
        be.check_status()
        n = 5
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            be.matmul_dev(dev, xd, y)
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / n
        flop = 2.0 * t * n_in * n_out
        out[f"m{t}"] = {"us": us, "tflops": flop / us / 1e6, "frac_of_bf16_peak": flop / us / 1e6 / peaks["bf16_tflops"],
                        "weight_gbs": n_out * n_in / us / 1e3, "frac_of_hbm_peak": n_out * n_in / us / 1e3 / peaks["hbm_gbs"]}
        del xd, y
    # ---- FP8 on both sides (b2_set_fp8_activations): activations quantized per token and per 128 k to e4m3, tcgen05 kind::f8f6f4,
    # bf16 output, as the configuration states it. The FP8 peak is measured here: an 8192^3 e4m3 x e4m3 torch._scaled_mm.
    try:
        a8 = torch.randn((8192, 8192), device="cuda").to(torch.float8_e4m3fn)
        b8 = torch.randn((8192, 8192), device="cuda").to(torch.float8_e4m3fn).t()
        one = torch.ones((), device="cuda")
        for _ in range(3):
            torch._scaled_mm(a8, b8, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
        best = 1e9
        for _ in range(10):
            e0.record()
            torch._scaled_mm(a8, b8, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        fp8_peak = 2.0 * 8192 ** 3 / (best * 1e-3) / 1e12
        del a8, b8
    except Exception as e:   # no FP8 library GEMM in this torch: twice the bf16 figure as a labelled stand-in
        fp8_peak = None
        out["fp8_peak_error"] = str(e)
    out["fp8_peak_tflops"] = fp8_peak
    out["fp8_peak_source"] = "torch._scaled_mm 8192^3 e4m3 x e4m3, best of 10, measured in this run" if fp8_peak else "2 x the measured bf16 burst (stand-in)"
    peak8 = fp8_peak or 2.0 * peaks["bf16_tflops"]
    be.set_fp8_activations(True)
    try:
        for t in (128, 8192):
            xd = torch.randn((t, n_in), device="cuda", dtype=torch.bfloat16)
            y = torch.empty((t, n_out), device="cuda", dtype=torch.bfloat16)
            for _ in range(2):
                be.matmul_dev(dev, xd, y)
            torch.cuda.synchronize()
            be.check_status()
            n = 5
            e0.record()
            for _ in range(n):
                be.matmul_dev(dev, xd, y)
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / n
            flop = 2.0 * t * n_in * n_out
            out[f"w8a8_m{t}"] = {"us": us, "tflops": flop / us / 1e6, "frac_of_fp8_peak": flop / us / 1e6 / peak8,
                                 "frac_of_bf16_peak": flop / us / 1e6 / peaks["bf16_tflops"], "weight_gbs": n_out * n_in / us / 1e3,
                                 "frac_of_hbm_peak": n_out * n_in / us / 1e3 / peaks["hbm_gbs"],
                                 "kernels": "quantize_act_e4m3_kernel + gemm_f8_tc_kernel (tcgen05 kind::f8f6f4), bf16 output"}
            del xd, y
    finally:
        be.set_fp8_activations(False)
    dev.free()
    return out


def decode_extras(be, peaks, n_tokens=256, ctx=2048, n_layers=32, kv_f16=False, cpu_tokens=0, rank=0, world=1, dist=None, check_tokens=0,
                  e2e_tokens=0):
    """Config 2: greedy decode tok/s of a Llama-style decoder (hidden 4096, 32 q / 8 kv heads of 128, FFN 14336, vocab
    128256; Q4_K body, Q6_K head, Q8_0 embeddings) after a `ctx`-token cache, batch 1, through the decode plan
    (one CUDA graph launch per token, embedding lookup and argmax on the device). Random-init weights; every layer
    has its own device memory (the same random bytes, generated once, are uploaded per layer)."""
    import numpy as np

    from oxinfer_b200 import decode as D
    from oxinfer_b200 import synth

    cfg = dict(n_layers=n_layers, h=4096, nh=32, nkv=8, hd=128, inter=14336, vocab=128256)
    layers, final_norm, head, embed, shapes = synth.llama_weights(seed=0xB2000020, same_layers=True, **cfg)
    dev_layers, wbytes = [], 0
    for L in layers:
        d = {name: be.upload(L[name], *shapes[name]) for name in shapes}
        wbytes += sum(d[name].bytes() for name in shapes)
        d["ln_pre"], d["ln_post"] = L["ln_pre"], L["ln_post"]
        dev_layers.append(d)
    dhead = be.upload(head, cfg["vocab"], cfg["h"])
    dembed = be.upload(embed, cfg["vocab"], cfg["h"])
    lc = D.LlamaConfig(eps=1e-5, rope_theta=500000.0, rope_interleaved=True, **cfg)
    head_bytes = dhead.bytes()
    full_layers = dev_layers
    if world > 1:   # tensor parallel: this rank's row shards, activations exchanged by peer stores
        dev_layers, dhead_r = D.shard_llama(be, dev_layers, dhead, lc, rank, world)
        g = D.llama_graph(lc, dev_layers, final_norm, dhead_r, rank, world)
    else:
        g = D.llama_graph(lc, dev_layers, final_norm, dhead)
    max_len = ctx + n_tokens
    plan = D.decode_plan(be, g, max_len, kv_f16=kv_f16)
    if plan is None:
        raise RuntimeError("decode plan declined: " + be.last_declined)
    if world > 1:
        handles = [None] * world
        dist.all_gather_object(handles, plan.export_handle())
        plan.attach_peers(rank, world, handles)
    rng = np.random.default_rng(7)
    row = cfg["nkv"] * cfg["hd"]
    per = row // world
    kv_rows = []
    # N > 1: rank 0 also holds the one-GPU plan over the unsharded weights (the shards are views into the same uploads) and
    # decodes a few tokens with it from the same cache: the tensor-parallel plan must produce the same tokens
    single = None
    if world > 1 and check_tokens and rank == 0:
        single = D.decode_plan(be, D.llama_graph(lc, full_layers, final_norm, dhead), ctx + check_tokens, kv_f16=kv_f16)
    for li in range(n_layers):   # the prefilled cache: unit-variance keys and values (a rank keeps its KV heads' columns)
        k = rng.standard_normal((ctx, row), dtype=np.float32)
        v = rng.standard_normal((ctx, row), dtype=np.float32)
        plan.kv_write(li, 0, np.ascontiguousarray(k[:, rank * per:(rank + 1) * per]), np.ascontiguousarray(v[:, rank * per:(rank + 1) * per]))
        if single is not None:
            single.kv_write(li, 0, k, v)
        if cpu_tokens and li == 0:
            kv_rows = [k, v]
    inv_freq = D.rope_inv_freq(cfg["hd"], lc.rope_theta)
    table = np.stack([D.rope_table(ctx + i, inv_freq) for i in range(n_tokens)])
    if world > 1:   # the ranks enter every collective step together (rank 0 has just built and filled a second plan)
        dist.barrier()
    warm_toks, _ = plan.generate(dembed, 1, ctx, min(8, n_tokens), table[: min(8, n_tokens)])    # warm-up (captures the graph)
    parity = None
    if world > 1 and check_tokens:
        nchk = min(check_tokens, 8, n_tokens)
        flag = 1
        if single is not None:
            ref_toks, _ = single.generate(dembed, 1, ctx, nchk, table[:nchk])
            flag = int(np.array_equal(ref_toks[:nchk], warm_toks[:nchk]))
            single.close()
        import torch

        ft = torch.tensor([flag], device="cuda", dtype=torch.int32)
        dist.all_reduce(ft, op=dist.ReduceOp.MIN)
        parity = f"first {nchk} greedy tokens equal the one-GPU plan's" if int(ft.item()) == 1 else "TOKEN MISMATCH against the one-GPU plan"
    times = []
    for _ in range(3):
        if world > 1:
            dist.barrier()
        toks, ms = plan.generate(dembed, 1, ctx, n_tokens, table)
        if world > 1:   # the slowest rank's device time
            import torch

            t = torch.tensor([ms], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        times.append(ms)
    ms = sorted(times)[1]
    kv_el = 2 if kv_f16 else 4
    kv_bytes = n_layers * 2 * (ctx + (n_tokens + 1) / 2) * row * kv_el
    algo = wbytes + head_bytes + cfg["h"] * 34 // 32 + kv_bytes   # whole job (all ranks together)
    out = {"tok_s": n_tokens / (ms * 1e-3), "ms_per_token": ms / n_tokens, "tokens": n_tokens, "context": ctx, "layers": n_layers, "n_gpus": world,
           "parallelism": f"tp{world}: row shards, 4 exchanges per layer by peer stores over NVLink" if world > 1 else "single GPU",
           "kv_cache": "f16" if kv_f16 else "f32", "launches_per_token": plan.launches_per_step() + 2,
           "bytes_per_token": int(algo), "gbs": algo / (ms / n_tokens * 1e-3) / 1e9,
           "frac_of_hbm_peak": algo / (ms / n_tokens * 1e-3) / 1e9 / (peaks["hbm_gbs"] * world),
           "distinct_tokens": int(len(set(toks.tolist()))), "timing": "CUDA events around the token loop, median of 3"}
    if parity is not None:
        out["parity"] = parity
    gbs = algo / (ms / n_tokens * 1e-3) / 1e9
    out["roofline"] = {"kernel": "one decode token: the plan's whole launch list (products, attention, norms)", "bound": "hbm", "achieved": gbs,
                       "peak": peaks["hbm_gbs"] * world, "unit": "GB/s", "frac": gbs / (peaks["hbm_gbs"] * world),
                       "frac_of_nominal_8000": gbs / (8000.0 * world), "traffic": None, "bytes_per_launch": int(algo),
                       "peak_source": f"copy bandwidth, {peaks['source']}"}
    e2e_tokens = min(e2e_tokens, n_tokens)
    if e2e_tokens and world == 1:
        # end to end through DecodePlan::step (b2_plan_step): per token the host hands over x and the RoPE row and reads the
        # hidden state and all logits back, takes the argmax and looks the next row up in a host table (as the reference's
        # generate loop does between steps, src/generate.rs)
        xs = np.random.default_rng(11).standard_normal((64, cfg["h"])).astype(np.float32)
        tok = 1
        plan.step(ctx, xs[0], table[0])
        t0 = time.perf_counter()
        for i in range(e2e_tokens):
            _, logits = plan.step(ctx + i, xs[tok % 64], table[i])
            tok = int(np.argmax(logits))
        dt = time.perf_counter() - t0
        out["e2e"] = {"value": e2e_tokens / dt, "unit": "tok/s", "tokens": e2e_tokens,
                      "h2d_bytes_per_step": int(4 * (cfg["h"] + table.shape[1])), "d2h_bytes_per_step": int(4 * (cfg["h"] + cfg["vocab"])),
                      "call": "b2_plan_step (DecodePlan::step): host x and RoPE row in, hidden + logits out, argmax on the host"}
    if cpu_tokens:
        # the reference's CPU decode path (oracle port) on the same model: a few tokens at the same context
        from oracle import oracle as O

        mats = {name: O.Matrix.gguf(O.Q4_K, layers[0][name].data, *shapes[name]) for name in shapes}
        cl = [dict(mats, ln_pre=L["ln_pre"], ln_post=L["ln_post"]) for L in layers]
        ocfg = O.LlamaCfg(n_layers, cfg["h"], cfg["nh"], cfg["nkv"], cfg["hd"], cfg["inter"], cfg["vocab"], 1, 1e-5, lc.scale)
        cpu = O.Llama(ocfg, cl, final_norm, O.Matrix.gguf(O.Q6_K, head.data, cfg["vocab"], cfg["h"]), ctx + cpu_tokens)
        for li in range(n_layers):
            cpu.kc[li, :ctx], cpu.vc[li, :ctx] = kv_rows[0], kv_rows[1]
        x = np.random.default_rng(1).standard_normal(cfg["h"]).astype(np.float32)
        t0 = time.perf_counter()
        for i in range(cpu_tokens):
            cpu.step(ctx + i, x, table[i], exact=False)
        dt = time.perf_counter() - t0
        out["cpu_baseline"] = {"value": cpu_tokens / dt, "unit": "tok/s", "cores": O.cpu_threads(), "kind": "port",
                               "sample": f"{cpu_tokens} tokens at context {ctx} (int8-activation decode kernels, f32 attention)"}
    if world == 1 and e2e_tokens:
        # Steps of several tokens (Backend::decode_plan_multi: speculative verification), through b2_plan_step_multi with host
        # buffers: t embeddings and RoPE rows in, t hidden states and t rows of logits out. Each step is first checked against
        # one-token steps of the plan above (bit for bit), then timed by the host clock around the synchronous calls.
        try:
            many = D.decode_plan_multi(be, g, max_len, 4, kv_f16=kv_f16)
            if many is None:
                raise RuntimeError("declined: " + be.last_declined)
            rng3 = np.random.default_rng(7)
            for li in range(n_layers):
                k = rng3.standard_normal((ctx, row), dtype=np.float32)
                v = rng3.standard_normal((ctx, row), dtype=np.float32)
                many.kv_write(li, 0, k, v)
                plan.kv_write(li, 0, k, v)
            xs = np.random.default_rng(12).standard_normal((4, cfg["h"])).astype(np.float32)
            ones = [plan.step(ctx + i, xs[i], table[i]) for i in range(4)]
            hm, lm = many.step_multi(ctx, xs, table[:4])
            same = all(np.array_equal(hm[i], ones[i][0]) and np.array_equal(lm[i], ones[i][1]) for i in range(4))
            res = {"parity": "4 tokens in one step: hidden states and logits equal four one-token steps bit for bit" if same
                   else "MISMATCH against one-token steps", "steps_timed": 24}
            for t in (1, 2, 3, 4):
                many.step_multi(ctx, xs[:t], table[:t])
                t0 = time.perf_counter()
                for _ in range(24):
                    many.step_multi(ctx, xs[:t], table[:t])
                dt = (time.perf_counter() - t0) / 24
                res[f"t{t}"] = {"ms_per_step": dt * 1e3, "tok_s": t / dt}
            res["call"] = "b2_plan_step_multi: host x [t][h] and RoPE rows in, hidden [t][h] and logits [t][vocab] out, synchronous"
            out["multi_token_steps"] = res
            many.close()
        except Exception as e:
            out["multi_token_steps"] = {"error": str(e)}
        # the same model with the products reading 16 of the activations' 21 bits (b2_set_fast_planes; not the default)
        try:
            be.set_fast_planes(True)
            fast = D.decode_plan(be, g, max_len, kv_f16=kv_f16)
            rng2 = np.random.default_rng(7)
            for li in range(n_layers):
                k = rng2.standard_normal((ctx, row), dtype=np.float32)
                v = rng2.standard_normal((ctx, row), dtype=np.float32)
                fast.kv_write(li, 0, k, v)
            fast.generate(dembed, 1, ctx, min(8, n_tokens), table[: min(8, n_tokens)])
            tf = sorted(fast.generate(dembed, 1, ctx, n_tokens, table)[1] for _ in range(3))[1]
            ftoks, _ = fast.generate(dembed, 1, ctx, n_tokens, table)
            same = 0
            while same < n_tokens and int(ftoks[same]) == int(toks[same]):
                same += 1
            out["fast_planes"] = {"tok_s": n_tokens / (tf * 1e-3), "ms_per_token": tf / n_tokens,
                                  "greedy_tokens_equal_to_default": f"first {same} of {n_tokens} (random-init weights: near-ties flip early)"}
            fast.close()
        except Exception as e:
            out["fast_planes"] = {"error": str(e)}
        finally:
            be.set_fast_planes(False)
    plan.close()
    return out


def gemm_format_extras(be, torch, peaks):
    """The prefill product at config 1's shape (512 x 4096 x 14336) in every format with a tensor-core kernel: the GEMM kernel
    alone (f16 activations used in place), weights larger than L2 (rotating copies), CUDA events around 20 launches."""
    from oxinfer_b200 import synth

    out = {}
    x16 = torch.from_numpy(synth.activations(M_TOK, K_IN, 78)).cuda().to(torch.float16)
    for fmt in ("q4_k", "mlx4", "q6_k", "q8_0", "f8_e4m3"):
        ref = synth.make(fmt, N_OUT, K_IN, 91)
        devs = [be.upload(ref, N_OUT, K_IN) for _ in range(6)]
        wbytes = devs[0].bytes()
        ys = [torch.empty((M_TOK, N_OUT), device="cuda") for _ in range(2)]
        for i in range(3):
            assert be.matmul_dev(devs[i % 6], x16, ys[i % 2])
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for i in range(20):
            be.matmul_dev(devs[i % 6], x16, ys[i % 2])
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) / 20 * 1e3
        out[fmt] = {"us": us, "tflops": FLOP_PER_STEP / us / 1e6, "frac_of_bf16_peak": FLOP_PER_STEP / us / 1e6 / peaks["bf16_tflops"],
                    "weight_bytes": wbytes, "rotating_copies": 6}
        for d in devs:
            d.free()
    be.check_status()
    return out


def prefill_extras(be, peaks, n_layers=32, tokens=2048, kv_f16=False):
    """Prefill of the config-2 model (Backend::decode_plan_prefill): `tokens` tokens per step from an empty cache, through
    b2_plan_step_multi with host buffers (embeddings and RoPE rows in, final-normed hidden states out). The device time is
    the step's kernels between the copies (CUDA events inside the call); the end-to-end time is the host clock around it."""
    import numpy as np

    from oxinfer_b200 import decode as D
    from oxinfer_b200 import synth

    cfg = dict(n_layers=n_layers, h=4096, nh=32, nkv=8, hd=128, inter=14336, vocab=128256)
    layers, final_norm, head, embed, shapes = synth.llama_weights(seed=0xB2000020, same_layers=True, **cfg)
    dev_layers = []
    for L in layers:
        d = {name: be.upload(L[name], *shapes[name]) for name in shapes}
        d["ln_pre"], d["ln_post"] = L["ln_pre"], L["ln_post"]
        dev_layers.append(d)
    dhead = be.upload(head, cfg["vocab"], cfg["h"])
    lc = D.LlamaConfig(eps=1e-5, rope_theta=500000.0, rope_interleaved=True, **cfg)
    inv_freq = D.rope_inv_freq(cfg["hd"], lc.rope_theta)
    pt = tokens
    pre = D.decode_plan_prefill(be, D.llama_graph(lc, dev_layers, final_norm, dhead, prefill=True), pt + 64, pt, kv_f16=kv_f16)
    if pre is None:
        raise RuntimeError("prefill plan declined: " + be.last_declined)
    one = D.decode_plan(be, D.llama_graph(lc, dev_layers, final_norm, dhead), 64, kv_f16=kv_f16)
    import torch

    # page-locked host buffers, as the headline's end-to-end figure uses
    xs_t = torch.from_numpy(np.random.default_rng(13).standard_normal((pt, cfg["h"])).astype(np.float32)).pin_memory()
    ptab_t = torch.from_numpy(np.stack([D.rope_table(i, inv_freq) for i in range(pt)])).pin_memory()
    hid_t = torch.empty((pt, cfg["h"]), dtype=torch.float32).pin_memory()
    xs, ptab, hid = xs_t.numpy(), ptab_t.numpy(), hid_t.numpy()
    # parity first: 48 tokens through the prefill plan and through one-token steps of the decode plan
    nchk = min(48, pt)
    hp, _ = pre.step_multi(0, xs[:nchk], ptab[:nchk])
    h1 = np.stack([one.step(i, xs[i], ptab[i], want_logits=False)[0] for i in range(nchk)])
    one.close()
    perr = float(np.max(np.max(np.abs(hp.astype(np.float64) - h1), axis=1) / np.maximum(np.max(np.abs(h1), axis=1), 1e-30)))
    res = {"tokens": pt, "layers": n_layers,
           "parity": f"{nchk} tokens: final hidden states within {perr:.2e} of one-token steps (row_err; bound 2e-3 per layer of depth)"}
    params = sum(shapes[name][0] * shapes[name][1] for name in shapes) * n_layers
    for t in sorted({pt, min(pt, 512), min(pt, 128)}, reverse=True):
        pre.step_multi(0, xs[:t], ptab[:t], hidden_out=hid[:t])
        dev, wall = [], []
        for _ in range(3):
            t0 = time.perf_counter()
            pre.step_multi(0, xs[:t], ptab[:t], hidden_out=hid[:t])
            wall.append(time.perf_counter() - t0)
            dev.append(pre.last_step_ms())
        dms, wms = sorted(dev)[1], sorted(wall)[1] * 1e3
        att = n_layers * cfg["nh"] * cfg["hd"] * 4 * (t * (t + 1) // 2)
        res[f"t{t}"] = {"device_ms": dms, "tok_s": t / (dms * 1e-3), "e2e_ms": wms, "e2e_tok_s": t / (wms * 1e-3),
                        "e2e_tflops": (2.0 * params * t + att) / (wms * 1e-3) / 1e12,
                        "tflops": (2.0 * params * t + att) / (dms * 1e-3) / 1e12,
                        "frac_of_bf16_sustained_peak": (2.0 * params * t + att) / (dms * 1e-3) / 1e12 / (peaks.get("bf16_tflops_sustained") or peaks["bf16_tflops"]),
                        "flop_products": 2.0 * params * t, "flop_attention": float(att), "launches": pre.launches_per_step()}
    res["call"] = "b2_plan_step_multi on a b2_decode_plan_prefill plan: x [t][h] and RoPE rows from page-locked host memory, hidden [t][h] back"
    res["h2d_bytes_per_step"] = int(4 * pt * (cfg["h"] + ptab.shape[1]))
    res["d2h_bytes_per_step"] = int(4 * pt * cfg["h"])
    pre.close()
    return res


def run_with_deadline(name, fn, seconds, stuck, rank=0):
    """fn() in a worker thread: its result, {"error": ...} if it raised, or, if it is still running after `seconds`, an error
    entry and `name` appended to `stuck` (the thread is a daemon: the caller prints what it has and leaves with os._exit)."""
    box = {}

    def work():
        try:
            box["out"] = fn()
        except Exception as e:
            box["out"] = {"error": str(e)}
            print(f"[bench rank {rank}] {name} failed: {e}", file=sys.stderr, flush=True)

    th = threading.Thread(target=work, daemon=True)
    th.start()
    th.join(seconds)
    if th.is_alive():
        stuck.append(name)
        print(f"[bench rank {rank}] {name} did not finish within {seconds} s", file=sys.stderr, flush=True)
        return {"error": f"did not finish within {seconds} s (a rank failed inside a collective step)"}
    return box["out"]


def run_b200(args, rank, world, local_rank):
    import numpy as np
    import torch

    import oxinfer_b200 as ob
    from oxinfer_b200 import synth

    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist

        # A rank that fails inside a collective section must end the run in minutes, not in the library's default half hour
        # (10 minutes of collective timeout and 8 of its heartbeat monitor): rank 0 then still prints what it has.
        import datetime

        os.environ.setdefault("TORCH_NCCL_HEARTBEAT_TIMEOUT_SEC", "60")
        os.environ.setdefault("TORCH_NCCL_DUMP_ON_TIMEOUT", "0")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank), timeout=datetime.timedelta(seconds=150))
    peaks = measured_peaks()
    be = ob.Backend(local_rank)
    stream = torch.cuda.current_stream()
    be.set_stream(stream.cuda_stream)

    if args.section == "gemv":
        emit(json.dumps({"extra": {"gemv": gemv_extras(be, torch, peaks, args.steps, args.case, not args.no_graph)}}))
        return
    if args.section in ("moe", "fp8"):
        fn = moe_extras if args.section == "moe" else fp8_extras
        emit(json.dumps({"extra": {args.section: fn(be, torch, peaks)}}))
        return
    if args.section == "refcuda":
        emit(json.dumps({"extra": {"reference_cuda": ref_cuda_extras(be, torch)}}))
        return
    if args.section == "gemm_formats":
        emit(json.dumps({"extra": {"gemm_formats": gemm_format_extras(be, torch, peaks)}}))
        return
    if args.section == "prefill":
        emit(json.dumps({"extra": {"prefill_plan": prefill_extras(be, peaks, args.layers, min(args.tokens, 8192) if args.tokens != 256 else 2048, args.kv_f16)}}))
        return
    if args.section == "decode":
        d = decode_extras(be, peaks, args.tokens, args.context, args.layers, args.kv_f16, rank=rank, world=world, dist=dist if world > 1 else None,
                          check_tokens=8 if world > 1 else 0, e2e_tokens=32 if world == 1 else 0)
        if rank == 0:
            emit(json.dumps({"extra": {"decode": d}}))
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return
    assert N_OUT % world == 0
    n_local = N_OUT // world
    full = synth.q4_k(N_OUT, K_IN, 1)        # the same matrix on every rank; a rank multiplies by its rows
    row_bytes = K_IN // 256 * 144
    ref = ob.Gguf(ob.FMT_Q4_K, np.ascontiguousarray(full.data[rank * n_local * row_bytes:(rank + 1) * n_local * row_bytes]))
    shard_bytes = ref.data.size
    copies = max(8, -(-2 * L2_BYTES // shard_bytes))  # rotate through > 2 x L2 of weights: every step streams from HBM
    devs = [be.upload(ref, n_local, K_IN) for _ in range(copies)]
    x_host = synth.activations(M_TOK, K_IN, 2)
    x_bf16 = torch.from_numpy(x_host).cuda().to(torch.bfloat16)
    x_f16 = torch.from_numpy(x_host).cuda().to(torch.float16)
    ycopies = 4
    ys = [torch.empty((M_TOK, n_local), device="cuda", dtype=torch.float32) for _ in range(ycopies)]
    y_full = torch.empty((world, M_TOK, n_local), device="cuda", dtype=torch.float32) if world > 1 else None

    # ---- N > 1: before anything is timed, this rank's shard against the same rows of the unsharded product ----
    parity = None
    peer_ok, peer_note = [False], [None]
    if world > 1:
        dfull = be.upload(full, N_OUT, K_IN)
        y_all = torch.empty((M_TOK, N_OUT), device="cuda", dtype=torch.float32)
        assert be.matmul_dev(dfull, x_bf16, y_all) and be.matmul_dev(devs[0], x_bf16, ys[0])
        torch.cuda.synchronize()
        be.check_status()
        same = torch.equal(y_all[:, rank * n_local:(rank + 1) * n_local].contiguous().view(torch.int32), ys[0].view(torch.int32))
        dist.all_gather_into_tensor(y_full, ys[0])
        torch.cuda.synchronize()
        same = same and torch.equal(y_full.permute(1, 0, 2).reshape(M_TOK, N_OUT).view(torch.int32), y_all.view(torch.int32))
        # the gather done by the GEMM's own epilogue (b2_matmul_sharded_peer): the library's communicator carries the buffers'
        # handles once; the result must equal the unsharded product bit for bit too
        try:
            box = [ob.Backend.comm_unique_id() if rank == 0 else None]
            dist.broadcast_object_list(box, src=0)
            be.comm_init(world, rank, box[0])
            be.comm_ready = True
            for i in range(3):
                yp = be.matmul_sharded_peer(devs[i % copies], x_bf16)
                if yp is None:
                    break
                torch.cuda.synchronize()
                be.check_status()
                same = same and torch.equal(yp.view(torch.int32), y_all.view(torch.int32)) if i == 0 else same
            peer_ok[0] = yp is not None
        except Exception as e:   # no NCCL, no peer access: the NCCL-through-torch gather stays
            peer_note[0] = str(e)
        agree = torch.tensor([1 if peer_ok[0] else 0], device="cuda", dtype=torch.int32)
        dist.all_reduce(agree, op=dist.ReduceOp.MIN)
        peer_ok[0] = int(agree.item()) == 1
        flag = torch.tensor([1 if same else 0], device="cuda", dtype=torch.int32)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        parity = "bit-identical" if int(flag.item()) == 1 else "MISMATCH"
        dfull.free()
        del y_all

    def step(i, gather=True):
        """gather: True = the fastest available way to leave the whole y on every rank, "nccl" = the library collective,
        False = none (y stays sharded)."""
        if world > 1 and gather is True and peer_ok[0]:
            assert be.matmul_sharded_peer(devs[i % copies], x_bf16) is not None
            return
        y = ys[i % ycopies]
        ok = be.matmul_dev(devs[i % copies], x_bf16, y)
        assert ok
        if world > 1 and gather:
            dist.all_gather_into_tensor(y_full, y)

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def timed(n, gather=True):
        """Device milliseconds of n steps, barrier + synchronize on both sides."""
        sync_all()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(n):
            step(i, gather)
        b.record()
        sync_all()
        return a.elapsed_time(b)

    warm = max(3, args.warmup)
    for i in range(warm):
        step(i)
    sync_all()
    be.check_status()
    # how many times the block of --steps steps must repeat for the timed region to hold 0.3 s of device time
    est_ms = timed(args.steps) / args.steps
    repeats = torch.tensor([max(1, int(-(-args.min_time_ms // (est_ms * args.steps))))], device="cuda", dtype=torch.int32)
    if world > 1:
        dist.all_reduce(repeats, op=dist.ReduceOp.MAX)
    repeats = int(repeats.item())

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    # ---- the GEMM kernel alone (f16 activations are used in place: one launch per call), a short burst before the long timed
    # region: the roofline's denominator is the burst peak, and after 0.3 s at the power cap the clocks are lower ----
    n_k = max(args.steps, 20)
    pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n_k)]
    for i in range(3):
        be.matmul_dev(devs[i % copies], x_f16, ys[i % ycopies])
    torch.cuda.synchronize()
    for i, (a, b) in enumerate(pairs):
        a.record()
        be.matmul_dev(devs[i % copies], x_f16, ys[i % ycopies])
        b.record()
    torch.cuda.synchronize()
    kern_ms = statistics.mean(a.elapsed_time(b) for a, b in pairs)
    # the same launches back to back with one pair of events around all of them: as dependent launches each one's set-up
    # (barriers, tensor memory, first weight copies) runs under its predecessor's epilogue, which an event between two
    # launches forbids; this is how the kernel runs inside a step, a prefill plan or a caller's loop
    ca, cb = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ca.record()
    for i in range(n_k):
        be.matmul_dev(devs[i % copies], x_f16, ys[i % ycopies])
    cb.record()
    torch.cuda.synchronize()
    chain_ms = ca.elapsed_time(cb) / n_k
    be.check_status()

    launches0 = be.launch_count()
    ms_total = timed(args.steps * repeats)
    launches = (be.launch_count() - launches0) // repeats
    be.check_status()
    ms_compute = timed(args.steps * repeats, gather=False) if world > 1 else ms_total
    ms_nccl = timed(args.steps * repeats, gather="nccl") if world > 1 and peer_ok[0] else ms_total

    # ---- end to end through the host-buffer call (b2_matmul): pinned x in, y out, every step ----
    xh = torch.from_numpy(x_host).pin_memory()
    yh = torch.empty((M_TOK, n_local), dtype=torch.float32).pin_memory()
    xh_np, yh_np = xh.numpy(), yh.numpy()
    e2e_steps = max(3, min(args.steps, 10))
    for i in range(2):
        assert be.matmul(xh_np, [ob.Job(devs[i % copies], yh_np)])
    sync_all()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2.record()
    for i in range(e2e_steps):
        assert be.matmul(xh_np, [ob.Job(devs[i % copies], yh_np)])
    e3.record()
    sync_all()
    e2e_ms_total = e2.elapsed_time(e3)
    clocks = sampler.stop() if rank == 0 else None

    t = torch.tensor([ms_total, e2e_ms_total, kern_ms, ms_compute, ms_nccl], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total, e2e_ms_total, kern_ms, ms_compute, ms_nccl = (float(v) for v in t.cpu())

    # The collective extras run in a worker thread with a deadline: if a rank fails inside one of them, the others would wait
    # in a collective until the process group's timeout aborts the process, and rank 0 would print nothing. With the deadline
    # the headline line is printed whatever happens to the extras, and the ranks then leave without the closing barrier.
    stuck = []

    def collective_section(name, fn, seconds=300):
        def on_device():
            torch.cuda.set_device(local_rank)
            with torch.cuda.stream(stream):
                return fn()

        return run_with_deadline(name, on_device, seconds, stuck, rank)

    dec_tp = None
    if world > 1 and args.section == "all":   # collective: every rank runs the tensor-parallel decode plan
        dec_tp = collective_section("tensor-parallel decode",
                                    lambda: decode_extras(be, peaks, 128, 2048, 32, False, rank=rank, world=world, dist=dist, check_tokens=8))
    ep = None
    if world > 1 and args.section == "all" and 128 % world == 0 and not stuck:   # collective: the expert-parallel MoE layer
        ep = collective_section("expert-parallel MoE", lambda: moe_ep_extras(be, torch, dist, rank, world))
    if rank == 0:
        n_timed = args.steps * repeats
        ms = ms_total / n_timed
        value = FLOP_PER_STEP / (ms * 1e-3) / 1e12
        e2e_ms = e2e_ms_total / e2e_steps
        kern_flop = FLOP_PER_STEP / world
        achieved = kern_flop / (kern_ms * 1e-3) / 1e12
        traffic, traffic_commit = profiled_traffic("gemm_q4k_tc_M512_K4096_N14336.txt") if world == 1 else (None, None)
        cfg = base_config(world)
        if parity is not None:
            cfg["parity"] = parity
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": warm, "repeats": repeats,
            "timed_region_ms": ms_total, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f16 operands, f32 accumulate", "data": "synthetic", "config": cfg,
            "step": (("x bf16 -> f16 conversion kernel + tcgen05 dequant-GEMM kernel on this rank's rows whose epilogue stores every tile into "
                      f"every rank's y ({M_TOK * N_OUT * 4 / 1e6:.0f} MB, bulk tensor stores over NVLink) + the ranks' meeting kernel"
                      if peer_ok[0] else
                      "x bf16 -> f16 conversion kernel + tcgen05 dequant-GEMM kernel on this rank's rows + NCCL all-gather of the f32 y "
                      f"({M_TOK * N_OUT * 4 / 1e6:.0f} MB) into rank-major blocks") if world > 1 else
                     "x bf16 -> f16 conversion kernel + tcgen05 dequant-GEMM kernel"),
            "inputs": f"{copies} weight copies ({copies * shard_bytes / 1e6:.0f} MB) and {ycopies} outputs in rotation",
            "e2e": {"value": FLOP_PER_STEP / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": int(xh.numel() * 4), "d2h_bytes_per_step": int(yh.numel() * 4) * world,
                    "call": "b2_matmul (Backend::matmul): pinned host f32 x in, f32 y out, synchronous"},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "roofline": {"kernel": "gemm_q4k_tc_kernel", "bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                         "frac": achieved / peaks["bf16_tflops"], "traffic": traffic,
                         "traffic_unit": "bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) read from profiles/gemm_q4k_tc_M512_K4096_N14336.txt"
                                         + (f", captured at {traffic_commit}" if traffic_commit else ""),
                         "us_per_launch": kern_ms * 1e3, "flop_per_launch": kern_flop, "peak_source": f"bf16 burst, {peaks['source']}",
                         "timing": "mean over launches that each sit between their own pair of CUDA events (the kernel's own duration, as ncu reports it)",
                         "chained": {"us_per_launch": chain_ms * 1e3, "achieved": kern_flop / (chain_ms * 1e-3) / 1e12,
                                     "frac": kern_flop / (chain_ms * 1e-3) / 1e12 / peaks["bf16_tflops"],
                                     "timing": "the same launches back to back between one pair of events (dependent launches overlap a launch's set-up "
                                               "with its predecessor's epilogue); rank 0's figure"}},
        }
        if world > 1:
            ms_c = ms_compute / n_timed
            line["compute_only"] = {"value": FLOP_PER_STEP / (ms_c * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_c,
                                    "note": "the same steps without the all-gather (y left sharded by columns on the ranks)"}
            if peer_ok[0]:
                ms_n = ms_nccl / n_timed
                line["nccl_gather"] = {"value": FLOP_PER_STEP / (ms_n * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_n,
                                       "note": "the same steps with the GEMM's result gathered by an NCCL all-gather instead of the epilogue's peer stores"}
            elif peer_note[0]:
                line["peer_store_unavailable"] = peer_note[0]
        if world == 1 and args.section == "all":
            from oracle import oracle as O

            threads = O.cpu_threads()
            times = cpu_prefill_tflops(threads, 2, 1)
            line["cpu_baseline"] = {"value": FLOP_PER_STEP / min(times) / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                                    "sample": "full workload (512 tokens x 14336 rows), best of 2 after 1 warm-up"}
            line["extra"] = {}
            for name, fn in (("gemv", lambda: gemv_extras(be, torch, peaks, 40)), ("moe", lambda: moe_extras(be, torch, peaks)),
                             ("fp8", lambda: fp8_extras(be, torch, peaks)), ("decode", lambda: decode_extras(be, peaks, cpu_tokens=2, e2e_tokens=32)),
                             ("prefill_plan", lambda: prefill_extras(be, peaks)),
                             ("gemm_formats", lambda: gemm_format_extras(be, torch, peaks)),
                             ("reference_cuda", lambda: ref_cuda_extras(be, torch))):
                try:
                    line["extra"][name] = fn()
                except Exception as e:  # the headline line must still print
                    line["extra"][name + "_error"] = str(e)
        if dec_tp is not None:
            line["extra"] = {"decode": dec_tp}
        if ep is not None:
            line.setdefault("extra", {})["moe_ep"] = ep
        line["summary"] = summarize(line)
        emit(json.dumps(line))
    if world > 1:
        if stuck:   # a worker thread still sits in a collective: no closing barrier, no orderly teardown
            sys.stdout.flush()
            os._exit(0)
        dist.barrier()
        dist.destroy_process_group()


def summarize(line: dict) -> dict:
    """The three parts of the metric in a few numbers, printed last so that the end of the line shows them."""
    out = {"gemm_tflops": round(line["value"], 1), "gemm_kernel_frac_of_bf16_peak": round(line["roofline"]["frac"], 3),
           "gemm_e2e_tflops": round(line["e2e"]["value"], 1)}
    ex = line.get("extra") or {}
    g = ex.get("gemv") or {}
    for key, short in (("mlx4_4096x4096", "gemv_cfg0_mlx4"), ("q4_k_14336x4096", "gemv_q4_k"), ("q6_k_32064x4096", "gemv_q6_k")):
        if key in g and "roofline" in g[key]:
            out[short + "_gbs"] = round(g[key]["roofline"]["achieved"], 0)
            out[short + "_frac_of_hbm"] = round(g[key]["roofline"]["frac"], 3)
    d = ex.get("decode") or {}
    if "tok_s" in d:
        out["decode_tok_s"] = round(d["tok_s"], 1)
        out["decode_frac_of_hbm"] = round(d["frac_of_hbm_peak"], 3)
        if "e2e" in d:
            out["decode_e2e_tok_s"] = round(d["e2e"]["value"], 1)
        if "parity" in d:
            out["decode_parity"] = d["parity"]
    pf = ex.get("prefill_plan") or {}
    if "t2048" in pf:
        out["prefill_2048_tok_s"] = round(pf["t2048"]["tok_s"], 0)
        out["prefill_2048_e2e_tok_s"] = round(pf["t2048"]["e2e_tok_s"], 0)
        out["prefill_2048_e2e_tflops"] = round(pf["t2048"]["e2e_tflops"], 0)
    mt = (d.get("multi_token_steps") or {}).get("t4")
    if mt:
        out["verify_4_tokens_ms"] = round(mt["ms_per_step"], 2)
    m = ex.get("moe") or {}
    for k in ("t1", "t64", "t512", "t4096"):
        if k in m:
            out["moe_" + k + "_us"] = round(m[k]["us"], 1)
    mep = ex.get("moe_ep") or {}
    for k in ("t512", "t4096"):
        if k in mep:
            out["moe_ep_" + k + "_us"] = round(mep[k]["us"], 1)
            out["moe_ep_parity"] = mep[k]["parity"]
    f = ex.get("fp8") or {}
    if "m8192" in f:
        out["fp8_m8192_tflops"] = round(f["m8192"]["tflops"], 0)
    if "w8a8_m8192" in f:
        out["fp8_w8a8_m8192_tflops"] = round(f["w8a8_m8192"]["tflops"], 0)
        out["fp8_w8a8_m8192_frac_of_fp8_peak"] = round(f["w8a8_m8192"]["frac_of_fp8_peak"], 3)
    return out


_OUT = None


def emit(text: str) -> None:
    """The result line goes to the process's original standard output; everything libraries print to file descriptor 1
    (NCCL's version banner, for one) is sent to standard error, so that standard output holds the JSON line alone."""
    global _OUT
    if _OUT is None:
        _OUT = sys.stdout
    _OUT.write(text + "\n")
    _OUT.flush()


def _keep_stdout_clean() -> None:
    global _OUT
    sys.stdout.flush()
    _OUT = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)


def main():
    _keep_stdout_clean()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--min-time-ms", type=float, default=300.0,
                    help="the block of --steps steps is repeated until the timed region holds this much device time (power / clock steady state)")
    ap.add_argument("--context", type=int, default=2048, help="with --section decode: tokens in the KV cache before the first decoded token")
    ap.add_argument("--case", default=None, help="with --section gemv: only the cases whose name contains this text")
    ap.add_argument("--no-graph", action="store_true", help="with --section gemv: host-launched kernels instead of a CUDA graph (profiling)")
    ap.add_argument("--layers", type=int, default=32, help="with --section decode: layers of the decoder (profiling runs use fewer)")
    ap.add_argument("--tokens", type=int, default=256, help="with --section decode: tokens to generate")
    ap.add_argument("--kv-f16", action="store_true", help="with --section decode: f16 KV caches instead of the reference's f32")
    ap.add_argument("--section", default="all", choices=["all", "gemm", "gemv", "decode", "prefill", "gemm_formats", "moe", "fp8", "refcuda"],
                    help="gemm: only the headline GEMM loops (no CPU baseline, no GEMV extras); gemv: only the GEMV extras (profiling runs)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    run_b200(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
