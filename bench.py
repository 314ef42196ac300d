#!/usr/bin/env python
"""Benchmark of the FP8 block-quantization hot path (one JSON line on stdout).

Headline workload (per GPU, weak scaling): the block-scaled FP8 GEMM forward of BASELINE.json configs[1]
    X bf16 [8192, 2048] ~ N(0,1)  --(1,128) e4m3-->  Xq      (timed, every step)
    W bf16 [2048, 8192] ~ N(0,0.02), quantized (128,128) once (the layer holds it quantized)
    Y = dq(Xq) . dq(Wq), fp32 accumulation, bf16 [8192, 8192]    (timed, every step)
A step is quantize(X) + GEMM; `value` is 2*M*N*K per step time, summed over ranks.
Synthetic seeded inputs; the step rotates over several input/output buffer sets so that every
step's data (201 MB per set, 800+ MB in rotation) comes from HBM, not from the 126 MB L2.

Beside the headline the line carries
    triple    (1 GPU)   configs[2]: forward + dgrad + wgrad with their quantizers at M = 32768, d_model 2048
    scaleout  (every N) configs[3]: the same triple at d_model 4096, FFN 16384, M = 65536 rows SPLIT over the
                        N GPUs (strong scaling, Student-t(3) activations, weights replicated, no collective)
    roofline_quantize / roofline_transposed / roofline_dequantize   the HBM-bound kernels on X[32768,2048]
    e2e       Linear.product with host buffers (X up, the quantized product down), with its copy-only ceiling

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
"""
from __future__ import annotations

import argparse
import json
import os
import re
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

M, N, K = 8192, 8192, 2048
FLOP_PER_STEP = 2 * M * N * K
QUANT_BYTES_PER_ELEM = 2 + 1 + 1 / 128 + 4 / 1024          # bf16 in, fp8 out, e8m0 per 128, fp32 per 1024
NBUF = 4
METRIC = "fp8_block_gemm_step_tflops"
WORKLOAD = "configs[1]: X[8192,2048] bf16 -> (1,128) e4m3; W[2048,8192] (128,128) e4m3; Y bf16 [8192,8192]"

# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) from the ncu captures summarised
# under profiles/.  Quantizer: profiles/quantize_row128_bf16_X16384x4096.md, the same 67.1 M elements as the
# X[32768,2048] launch timed here (134.2 MB read + 30.8 MB written before the kernel ends; the rest of the
# 67.9 MB output is written back from L2 later).  GEMM: the benchmark launch itself, second table of profiles/gemm_tn_pair_4096x4096x2048.md.
GEMM_DRAM_TRAFFIC_BYTES = 119.3e6
QUANT_DRAM_TRAFFIC_BYTES = 165.1e6


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()       # the exact child this object started
        self.thread.join(timeout=2)
        sm = [float(r[0]) for r in self.rows if len(r) >= 6 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 6 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 6 for n, v in zip(names, r[2:6]) if v.lower().startswith("active")})
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


# --------------------------------------------------------------------------- CPU reference arm
CPU_SAMPLE_ROWS = 2048      # a quarter of the workload's rows; W is the full [2048, 8192]


def cpu_sample(rows: int, seed: int = 0):
    """One pass of the oracle (numpy restatement of the reference) over a row sample of the
    workload: quantize X[rows, K], then dq(X) @ dq(W) in f32 for all N columns."""
    import numpy as np
    from oracle import qarr_oracle as oracle
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((rows, K)).astype(np.float32)
    w = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
    wq = oracle.quantize_impl(w, (128, 128))
    t0 = time.perf_counter()
    xq = oracle.quantize_impl(x, (1, 128))
    y = oracle.matmul_impl(*xq, *wq, (1, 128), (128, 128))
    dt = time.perf_counter() - t0
    return dt, float(np.abs(y).max())


def _blas_threads():
    try:
        from threadpoolctl import threadpool_info
        return max([int(p.get("num_threads", 1)) for p in threadpool_info()] or [1])
    except Exception:
        return None


def run_cpu_child(args):
    """The CPU pass proper, in a process whose BLAS thread count was set before numpy was imported (a
    launcher such as torchrun exports OMP_NUM_THREADS=1 to its ranks, which numpy's BLAS reads at import).
    `--steps K --warmup W`: W untimed passes, K timed ones; budget mode (--steps 0): passes for about 12 s."""
    rows = CPU_SAMPLE_ROWS
    for i in range(max(args.warmup, 1)):
        cpu_sample(rows, seed=100 + i)
    total, reps = 0.0, 0
    if args.steps > 0:
        for i in range(args.steps):
            total += cpu_sample(rows, seed=i)[0]       # the pass itself: inputs are generated and the weight quantized outside the clock, as on the GPU arm
        reps = args.steps
    else:
        while total < 12.0 and reps < 50:
            total += cpu_sample(rows, seed=reps + 1)[0]
            reps += 1
    print(json.dumps({"seconds": total, "passes": reps, "rows": rows, "threads": _blas_threads(), "cores": os.cpu_count()}))
    return 0


def cpu_pass(steps: int, warmup: int):
    env = dict(os.environ)
    for v in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS"):
        env[v] = str(os.cpu_count() or 1)
    r = subprocess.run([sys.executable, str(Path(__file__).resolve()), "--cpu-child", "--steps", str(steps), "--warmup", str(warmup)],
                       env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=900)
    if r.returncode != 0:
        raise RuntimeError(f"CPU pass failed: {r.stderr[-500:]}")
    return json.loads(r.stdout.strip().splitlines()[-1])


def cpu_baseline():
    c = cpu_pass(0, 1)
    per = c["seconds"] / c["passes"]
    return {"value": 2 * c["rows"] * N * K / per / 1e12, "unit": "TFLOP/s", "cores": c["cores"], "threads": c["threads"], "kind": "port",
            "sample": f"oracle (numpy+ml_dtypes restatement; jax is not installed, so the reference's own JAX CPU path cannot run): "
                      f"quantize X[{c['rows']},{K}] + dequantize both operands + f32 matmul to [{c['rows']},{N}], mean of {c['passes']} passes, "
                      f"numpy BLAS threads = {c['threads']}, elementwise part single-threaded"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    c = cpu_pass(max(args.steps, 1), args.warmup)
    rows, dt = c["rows"], c["seconds"]
    val = 2 * rows * N * K * c["passes"] / dt / 1e12
    cb = {"value": val, "unit": "TFLOP/s", "cores": c["cores"], "threads": c["threads"], "kind": "port",
          "sample": f"each step = oracle pass over a {rows}-row sample of X (quantize + dequantize + f32 matmul against the full W[{K},{N}]); "
                    f"run in a child process with the BLAS thread count set to all cores before numpy is imported"}
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt / c["passes"] * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": {"workload": WORKLOAD, "sample_rows": rows},
        "cpu_baseline": cb, "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))
    return 0


# --------------------------------------------------------------------------- the training triple (configs[2], configs[3])
def student_t3(shape, gen, device):
    """Student-t with 3 degrees of freedom from seeded normals: z / sqrt(chi2_3 / 3)."""
    import torch
    z = torch.randn(shape, device=device, generator=gen)
    chi = torch.zeros(shape, device=device)
    for _ in range(3):
        chi += torch.randn(shape, device=device, generator=gen) ** 2
    return z / (chi / 3.0).sqrt()


def time_triple(tokens: int, d_model: int, ffn: int, dist: str, seed: int, reps: int, sync):
    """forward + dgrad + wgrad of the six projections of one block (4 x [d,d], [d,ffn], [ffn,d]) on `tokens` rows with
    their quantizers: per projection quantize_dual(x) -> fwd GEMM (bf16 Y), quantize_dual(dY) -> dgrad GEMM (bf16 dX)
    and wgrad GEMM (f32 dW, contraction over the tokens).  Weights are held quantized (quantized once, outside the
    clock, as the layer holds them).  Returns milliseconds per triple (all six projections) with and without the
    quantizers, timed with CUDA events after warm-up; `sync` is called on both sides of each timed region."""
    import torch
    from pratchya_b200 import _lib
    from pratchya_b200._qualia import _ops
    lib = _lib.load()
    dev = torch.device("cuda", torch.cuda.current_device())
    stream = torch.cuda.current_stream().cuda_stream
    gen = torch.Generator(device=dev).manual_seed(seed)
    op = _ops._operand
    shapes = [(d_model, d_model), (d_model, ffn), (ffn, d_model)]
    counts = [4, 1, 1]
    total_ms, gemm_ms, per_shape = 0.0, 0.0, {}
    for (k_in, n_out), count in zip(shapes, counts):
        x = (student_t3((tokens, k_in), gen, dev) if dist == "student_t" else torch.randn(tokens, k_in, device=dev, generator=gen)).to(torch.bfloat16)
        dy = (torch.randn(tokens, n_out, device=dev, generator=gen) * 1e-3).to(torch.bfloat16)
        w = (torch.randn(k_in, n_out, device=dev, generator=torch.Generator(device=dev).manual_seed(7 + k_in + n_out)) * 0.02).to(torch.bfloat16)
        wq = _ops.quantize_impl(w, (128, 128))
        wt = _ops.transpose_bytes(wq[0])

        def gemms(xq, xt, gq, gt):
            y = _ops.gemm_tn(op(xq[0], xq[1], xq[2], tokens, k_in, (1, 128)), op(wt, wq[1], wq[2], n_out, k_in, (128, 128), 1), torch.bfloat16, dev)
            dx = _ops.gemm_tn(op(gq[0], gq[1], gq[2], tokens, n_out, (1, 128)), op(wq[0], wq[1], wq[2], k_in, n_out, (128, 128)), torch.bfloat16, dev)
            dw = _ops.gemm_tn(op(xt[0], xt[1], xt[2], k_in, tokens, (1, 128)), op(gt[0], gt[1], gt[2], n_out, tokens, (1, 128)), torch.float32, dev)
            return y, dx, dw

        def full():
            xq, xt = _ops.quantize_dual_impl(x)
            gq, gt = _ops.quantize_dual_impl(dy)
            return gemms(xq, xt, gq, gt)

        def timed(fn):
            for _ in range(2):
                fn()
            sync()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(reps):
                fn()
            b.record()
            sync()
            _lib.check(lib.pb_gemm_check(stream))
            return a.elapsed_time(b) / reps

        t_full = timed(full)
        xq, xt = _ops.quantize_dual_impl(x)
        gq, gt = _ops.quantize_dual_impl(dy)
        t_gemm = timed(lambda: gemms(xq, xt, gq, gt))
        per_shape[f"{k_in}->{n_out}"] = {"ms": t_full, "gemm_ms": t_gemm, "tflops": 6.0 * tokens * k_in * n_out / t_full / 1e9,
                                         "gemm_tflops": 6.0 * tokens * k_in * n_out / t_gemm / 1e9}
        total_ms += count * t_full
        gemm_ms += count * t_gemm
        del x, dy, w, wq, wt, xq, xt, gq, gt
        torch.cuda.empty_cache()
    flop = 6.0 * tokens * (4 * d_model * d_model + 2 * d_model * ffn)
    return {"ms": total_ms, "gemm_ms": gemm_ms, "flop": flop, "per_projection": per_shape}


# --------------------------------------------------------------------------- the end-to-end training step (configs[4])
def time_model_step(world: int, rank: int, dev, barrier, host_group=None, steps: int = 2):
    """One data-parallel training step of the modified RWKV-7 model with every linear layer on the FP8 path: 24 layers,
    d_model 2048, head size 64, vocabulary 65536, context 4096, 8 sequences per GPU (the configuration's global batch of
    64 at 8 GPUs) of random token ids, random-init f32 master weights.  A step = forward + backward + all-reduce of the
    gradients in bf16 over NCCL + a sign-momentum update of the masters.  The reference recomputes every block in the
    backward pass (nnx.remat); here as many of the last blocks as the GPU's free memory holds keep their activations
    instead (10 GB per block at 8 x 4096 tokens, with 20 GB left free) and the others are recomputed: same loss and
    gradient bits, one forward pass less for the kept blocks.  CUDA events around each step, barrier on both sides,
    mean of `steps` after two warm-up steps.

    With more than one rank every step ends its own GPU work (a synchronize) and the ranks then agree on the host, through
    `host_group` (gloo, CPU tensors), that all of them are healthy before any of them enters the gradient exchange: a rank
    whose GPU work failed says so there, and all ranks return an error record with no collective in flight."""
    import torch
    import torch.distributed as dist
    from pratchya_b200._nnx_impl._model import PratchyaConfig
    from pratchya_b200._qualia import set_literal_dot_precision
    set_literal_dot_precision("tf32")   # the (128,1)-grid layers' backward dots (LoRA, lm_head): what an f32 dot gets under XLA on a GPU
    cfg = PratchyaConfig()
    seqs, ctx = 8, 4096
    torch.cuda.empty_cache()
    free_bytes, _ = torch.cuda.mem_get_info(dev)
    # measured: a step with every block recomputed peaks at 35 GB (the logits' cotangent written over the logits), and a block that
    # keeps its activations adds 10.1 GB
    kept = torch.tensor([max(0, min(cfg.n_layers, int((free_bytes - 37e9 - 20e9) // (10.1e9 * seqs * ctx / 32768))))], dtype=torch.int32)
    if world > 1:
        dist.all_reduce(kept, op=dist.ReduceOp.MIN, group=host_group)
    kept = int(kept.item())
    gen = torch.Generator(device=dev).manual_seed(100 + rank)
    ids = torch.randint(0, cfg.vocab_size, (seqs, ctx), device=dev, generator=gen)
    out = None
    for attempt_kept in ([kept, 0] if kept else [0]):
        out = _model_step_once(cfg, attempt_kept, world, rank, dev, barrier, host_group, steps, ids, seqs, ctx)
        if "error" not in out or not out.get("retry"):
            break
    out.pop("retry", None)
    try:
        set_literal_dot_precision("f32")
    except Exception:      # noqa: BLE001
        pass
    return out


class _StepFailed(RuntimeError):
    pass


def _model_step_once(cfg, kept, world, rank, dev, barrier, host_group, steps, ids, seqs, ctx):
    import torch
    import torch.distributed as dist
    from pratchya_b200._nnx_impl._dp import agree_on_health, allreduce_gradients, run_guarded
    from pratchya_b200._nnx_impl._model import PratchyaCausalLM

    def agree(code: int) -> int:       # the worst of the ranks' codes (0 healthy, 1 out of memory, 2 any other failure)
        return agree_on_health(code, world, host_group)

    def guarded(fn):                   # fn, then this rank's GPU work to its end; (code, message)
        return run_guarded(fn, lambda: torch.cuda.synchronize(dev))

    state = {}

    def build():
        state["model"] = PratchyaCausalLM(cfg, seed=11, device=dev, remat=cfg.n_layers - kept)
        state["params"] = [p for p in state["model"].parameters()]
        state["momentum"] = [torch.zeros_like(p) for p in state["params"]]
        torch.cuda.reset_peak_memory_stats(dev)

    losses = []

    def compute():
        for p in state["params"]:
            p.grad = None
        _, loss = state["model"](ids, ids, keep_logits=False)
        loss.backward()
        losses.append(loss.detach())

    def finish(exchange):
        params, momentum = state["params"], state["momentum"]
        if world > 1 and exchange:
            allreduce_gradients(params, world)
        grads = [p.grad for p in params]
        with torch.no_grad():
            torch._foreach_mul_(momentum, 0.9)
            torch._foreach_add_(momentum, grads, alpha=0.1)
            torch._foreach_add_(params, [m.sign() for m in momentum], alpha=-1e-4)

    def step(exchange=True):
        code, msg = guarded(compute)
        worst = agree(code)
        if worst:
            raise _StepFailed(msg or "another rank failed", worst)
        finish(exchange)

    def failed(msg, worst):
        for p in state.get("params", []):
            p.grad = None
        state.clear()
        if worst == 1:
            try:
                torch.cuda.empty_cache()
            except Exception:      # noqa: BLE001
                pass
        return {"error": msg, "kept_blocks": kept, "retry": worst == 1 and kept > 0}

    code, msg = guarded(build)
    worst = agree(code)
    if worst:
        return failed(msg or "another rank failed while building the model", worst)
    try:
        step(exchange=False)     # the first warm-up step without the exchange
        step()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        barrier()
    except _StepFailed as e:
        return failed(e.args[0], e.args[1])
    ms = e0.elapsed_time(e1) / steps
    n_params = sum(p.numel() for p in state["params"])
    out = {"ms_per_step": ms, "tokens_per_gpu": seqs * ctx, "parameters": n_params, "losses": [float(l) for l in losses],
           "peak_memory_gb": torch.cuda.max_memory_allocated(dev) / 1e9, "literal_dot_precision": "tf32",
           "recomputed_blocks": cfg.n_layers - kept, "kept_blocks": kept}
    state.clear()
    torch.cuda.empty_cache()
    return out


# --------------------------------------------------------------------------- GPU arm
def gpu_cpu_affinity(index: int):
    """The CPU set `nvidia-smi topo -m` lists for this GPU (read only), or None."""
    try:
        out = subprocess.run(["nvidia-smi", "topo", "-m"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True, timeout=20).stdout
    except (OSError, subprocess.TimeoutExpired):
        return None
    for line in out.splitlines():
        if re.match(rf"\s*GPU{index}\s", line):
            m = re.search(r"\s(\d+(?:-\d+)?(?:,\d+(?:-\d+)?)*)\s+(\d+|N/A)\s", line + " ")
            if not m:
                return None
            cpus = set()
            for part in m.group(1).split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
            return cpus
    return None


def run_ours(args):
    import torch
    import torch.distributed as dist
    from pratchya_b200 import _lib
    from pratchya_b200._qualia import _ops
    from pratchya_b200._nnx_impl import Linear

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the pratchya_b200 ops have no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    # pinned host buffers are allocated by a process that sits on the CPUs next to its GPU
    affinity = gpu_cpu_affinity(local)
    if affinity:
        try:
            os.sched_setaffinity(0, affinity & os.sched_getaffinity(0) or os.sched_getaffinity(0))
        except OSError:
            affinity = None
    host_group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        # a second group on CPU tensors: the ranks agree through it, step by step, that every one of them is still healthy before
        # they enter a collective of the end-to-end step, so that a rank whose GPU work failed leaves between steps with nothing in flight
        host_group = dist.new_group(backend="gloo")
    lib = _lib.load()
    stream = torch.cuda.current_stream().cuda_stream

    gen = torch.Generator(device=dev).manual_seed(1234 + rank)       # each rank owns its own row shard
    xs = [torch.randn(M, K, device=dev, generator=gen, dtype=torch.float32).to(torch.bfloat16) for _ in range(NBUF)]
    w = (torch.randn(K, N, device=dev, generator=torch.Generator(device=dev).manual_seed(7), dtype=torch.float32) * 0.02).to(torch.bfloat16)
    layer = Linear(K, N, (128, 128), kernel=w)                       # weight quantized once, replicated on every rank
    wq, w_s8, w_s32 = layer.kernel.get_value(), layer.kernel.sc_fp8, layer.kernel.sc_fp32
    w_t = layer.kernel.transposed_value()

    # preallocated device buffers: the timed loop calls the C ABI only
    xq = [torch.empty(M, K, device=dev, dtype=torch.uint8) for _ in range(NBUF)]
    x_s8 = [torch.empty(M * K // 128, device=dev, dtype=torch.uint8) for _ in range(NBUF)]
    x_s32 = [torch.empty(M * K // 1024, device=dev, dtype=torch.float32) for _ in range(NBUF)]
    ys = [torch.empty(M, N, device=dev, dtype=torch.bfloat16) for _ in range(NBUF)]
    ops_a = [_lib.Operand(xq[i].data_ptr(), x_s8[i].data_ptr(), x_s32[i].data_ptr(), M, K, 1, 128, _lib.PB_E4M3, 0) for i in range(NBUF)]
    op_b = _lib.Operand(w_t.data_ptr(), w_s8.data_ptr(), w_s32.data_ptr(), N, K, 128, 128, _lib.PB_E4M3, 1)
    ws_bytes = lib.pb_gemm_workspace_size(ops_a[0], op_b)
    ws = torch.empty(ws_bytes, device=dev, dtype=torch.uint8)

    # The step is Linear.__call__'s product: quantize the activation (the quantizer also lays its
    # scales out for the GEMM), then the GEMM.  The weight's scales are laid out by the first
    # (warm-up) call and reused: they do not change between steps.
    b_ready = [0]

    def quantize(i):
        _lib.check(lib.pb_quantize_for_gemm(xs[i].data_ptr(), _lib.PB_BF16, M, K, _lib.PB_E4M3,
                                            xq[i].data_ptr(), x_s8[i].data_ptr(), x_s32[i].data_ptr(),
                                            op_b, ws.data_ptr(), ws_bytes, stream))

    def gemm(i):
        _lib.check(lib.pb_gemm_tn_ex(ops_a[i], op_b, ys[i].data_ptr(), _lib.PB_BF16, N, ws.data_ptr(), ws_bytes,
                                     _ops.GEMM_A_PREPARED | b_ready[0], stream))
        b_ready[0] = _ops.GEMM_B_PREPARED

    def step(i):
        quantize(i % NBUF)
        gemm(i % NBUF)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(max(args.warmup, 3)):
        step(i)
    barrier()
    _lib.check(lib.pb_gemm_check(stream))

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.15)
    # The timed region replays a CUDA graph of NBUF consecutive steps (the library's calls are stream-ordered
    # and allocate nothing, so they capture as they are); K steps that are not a multiple of NBUF run eagerly.
    graph = None
    if args.steps % NBUF == 0:
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream())
        main_stream = stream
        with torch.cuda.stream(side):
            stream = side.cuda_stream
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for i in range(NBUF):
                    step(i)
            stream = main_stream
        torch.cuda.current_stream().wait_stream(side)
        graph.replay()
        torch.cuda.synchronize()
        _lib.check(lib.pb_gemm_check(stream))
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t0.record()
    if graph is not None:
        for _ in range(args.steps // NBUF):     # the timed region: K steps, nothing else on the stream
            graph.replay()
    else:
        for i in range(args.steps):
            step(i)
    t1.record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    total_ms = t0.elapsed_time(t1)
    _lib.check(lib.pb_gemm_check(stream))

    # the same K steps once more with an event after every launch, for the per-kernel durations
    # (an event between two launches costs the step ~6 %, so it stays out of the timed region)
    n_parts = min(args.steps, 200)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2 * n_parts + 1)]
    ev[0].record()
    for i in range(n_parts):
        quantize(i % NBUF)
        ev[2 * i + 1].record()
        gemm(i % NBUF)
        ev[2 * i + 2].record()
    barrier()
    q_ms = statistics.mean(ev[2 * i].elapsed_time(ev[2 * i + 1]) for i in range(n_parts))
    g_ms = statistics.mean(ev[2 * i + 1].elapsed_time(ev[2 * i + 2]) for i in range(n_parts))
    _lib.check(lib.pb_gemm_check(stream))

    # ---- the HBM-bound kernels alone on the largest activation of the training configs (202 MB per launch)
    qm, qk = 32768, 2048
    big = [torch.randn(qm, qk, device=dev, dtype=torch.bfloat16) for _ in range(2)]
    bq = torch.empty(qm, qk, device=dev, dtype=torch.uint8)
    b8 = torch.empty(qm * qk // 128, device=dev, dtype=torch.uint8)
    b32 = torch.empty(qm * qk // 1024, device=dev, dtype=torch.float32)
    bqt = torch.empty(qk, qm, device=dev, dtype=torch.uint8)
    back = [torch.empty(qm, qk, device=dev, dtype=torch.bfloat16) for _ in range(2)]
    tws_bytes = lib.pb_quantize_transposed_workspace_size(1, qm, qk, 128)
    tws = torch.empty(max(tws_bytes, 16), device=dev, dtype=torch.uint8)

    def big_quant(i):
        _lib.check(lib.pb_quantize(big[i % 2].data_ptr(), _lib.PB_BF16, 1, qm, qk, 1, 128, _lib.PB_E4M3,
                                   bq.data_ptr(), b8.data_ptr(), b32.data_ptr(), None, 0, stream))

    def big_quant_t(i):
        _lib.check(lib.pb_quantize_transposed(big[i % 2].data_ptr(), _lib.PB_BF16, 1, qm, qk, 128, _lib.PB_E4M3,
                                              bqt.data_ptr(), b8.data_ptr(), b32.data_ptr(), tws.data_ptr(), tws_bytes, stream))

    def big_dequant(i):
        _lib.check(lib.pb_dequantize(bq.data_ptr(), _lib.PB_E4M3, b8.data_ptr(), b32.data_ptr(), 1, qm, qk, 1, 128,
                                     _lib.PB_BF16, back[i % 2].data_ptr(), stream))

    def time_alone(fn, reps=20):
        for i in range(3):
            fn(i)
        torch.cuda.synchronize()
        e = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        e[0].record()
        for i in range(reps):
            fn(i)
        e[1].record()
        torch.cuda.synchronize()
        return e[0].elapsed_time(e[1]) / reps

    big_qt_ms = time_alone(big_quant_t)
    big_q_ms = time_alone(big_quant)          # leaves the row form's triple in (bq, b8, b32) for the dequantizer
    big_dq_ms = time_alone(big_dequant)
    quant_bytes = qm * qk * QUANT_BYTES_PER_ELEM
    del big, back
    # the same token-major quantizer on f32 input (the end-to-end model's activations are f32): 4 + 1 + scales bytes per element
    big32 = [torch.randn(qm, qk, device=dev, dtype=torch.float32) for _ in range(2)]

    def big_quant_t32(i):
        _lib.check(lib.pb_quantize_transposed(big32[i % 2].data_ptr(), _lib.PB_F32, 1, qm, qk, 128, _lib.PB_E4M3,
                                              bqt.data_ptr(), b8.data_ptr(), b32.data_ptr(), tws.data_ptr(), tws_bytes, stream))

    big_qt32_ms = time_alone(big_quant_t32)
    quant32_bytes = qm * qk * (QUANT_BYTES_PER_ELEM + 2.0)
    _lib.check(lib.pb_gemm_check(stream))
    del big32, bq, bqt, tws

    if args.headline_only:
        if rank == 0:
            print(json.dumps({"metric": METRIC, "value": world * FLOP_PER_STEP / (total_ms / args.steps * 1e-3) / 1e12, "unit": "TFLOP/s",
                              "n_gpus": world, "steps": args.steps, "ms_per_step": total_ms / args.steps, "gemm_ms": g_ms, "quantize_ms": q_ms,
                              "quantize_alone_us": big_q_ms * 1e3, "transposed_alone_us": big_qt_ms * 1e3, "dequantize_alone_us": big_dq_ms * 1e3,
                              "note": "--headline-only: a reduced line for profiler runs, not the benchmark line"}))
        if world > 1:
            dist.destroy_process_group()
        return 0

    # ---- end to end through the public API with host buffers: every step copies its X from pinned host
    # memory, runs Linear.product (quantize, GEMM, and the (1,128) re-quantization of the product that the
    # reference's `x_q @ kernel` returns), and copies that quantized product -- bytes and both scale arrays --
    # back to pinned host memory.  Copies run on their own streams over two buffer sets, so step i+1's
    # upload and step i-1's download overlap step i's kernels; the same copies without any kernel give
    # the ceiling the host side allows.
    x_host = [x.cpu().pin_memory() for x in xs[:2]]
    yq_host = [torch.empty(M, N, dtype=torch.uint8).pin_memory() for _ in range(2)]
    y8_host = [torch.empty(M * N // 128, dtype=torch.uint8).pin_memory() for _ in range(2)]
    y32_host = [torch.empty(M * N // 1024, dtype=torch.float32).pin_memory() for _ in range(2)]
    x_dev = [torch.empty(M, K, device=dev, dtype=torch.bfloat16) for _ in range(2)]
    d2h_bytes = M * N + M * N // 128 + 4 * (M * N // 1024)
    cur = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    in_ready = [torch.cuda.Event() for _ in range(2)]
    cmp_done = [torch.cuda.Event() for _ in range(2)]
    out_done = [torch.cuda.Event() for _ in range(2)]
    last = [None, None]

    def download(b, yq):
        yq_host[b].copy_(yq.get_value().view(torch.uint8), non_blocking=True)
        y8_host[b].copy_(yq.sc_fp8.view(torch.uint8).reshape(-1), non_blocking=True)
        y32_host[b].copy_(yq.sc_fp32.reshape(-1), non_blocking=True)

    def e2e_step(i, compute=True):
        b = i % 2
        with torch.cuda.stream(s_in):
            s_in.wait_event(cmp_done[b])            # the kernels of step i-2 have read x_dev[b]
            x_dev[b].copy_(x_host[b], non_blocking=True)
            in_ready[b].record(s_in)
        cur.wait_event(in_ready[b])
        if compute:
            last[b] = layer.product(x_dev[b])
        yq = last[b]
        cmp_done[b].record(cur)
        with torch.cuda.stream(s_out):
            s_out.wait_event(cmp_done[b])
            s_out.wait_event(out_done[b])           # the host buffers of step i-2 have been written
            download(b, yq)
            out_done[b].record(s_out)
        for t in (yq.get_value(), yq.sc_fp8, yq.sc_fp32):
            t.record_stream(s_out)

    e2e_steps = max(4, min(args.steps, 10))

    def e2e_time(compute):
        for i in range(2):
            e2e_step(i, compute)
        cur.wait_stream(s_out)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(e2e_steps):
            e2e_step(i, compute)
        cur.wait_stream(s_in)
        cur.wait_stream(s_out)
        e1.record()
        barrier()
        return e0.elapsed_time(e1) / e2e_steps

    # median of five passes: the host side of these copies (shared PCIe switch, other tenants) is noisy
    e2e_runs = [e2e_time(True) for _ in range(5)]
    e2e_ms = statistics.median(e2e_runs)
    copy_only_ms = statistics.median(e2e_time(False) for _ in range(3))
    _lib.check(lib.pb_gemm_check(stream))

    # ---- the training triple: configs[2] on one GPU, and configs[3] split by rows over all the ranks
    def local_sync():
        torch.cuda.synchronize()

    triple = time_triple(32768, 2048, 8192, "normal", 99, reps=5, sync=local_sync) if world == 1 else None
    so_tokens, so_d, so_ffn = 65536, 4096, 16384
    scale = time_triple(so_tokens // world, so_d, so_ffn, "student_t", 500 + rank, reps=3, sync=barrier)
    one_gpu = scale if world == 1 else None
    if world > 1:
        # rank 0 alone repeats the whole 65536-row job, so that the line carries its own 1-GPU time
        barrier()
        if rank == 0:
            one_gpu = time_triple(so_tokens, so_d, so_ffn, "student_t", 500, reps=2, sync=local_sync)
        barrier()

    # ---- the one collective of the end-to-end step (configs[4]): the data-parallel all-reduce of the gradients,
    # plain NCCL over NVLink.  The quantize / GEMM path above has no collective; this times the exchange that a
    # 24-layer d_model-2048 model (1.48 G parameters, bf16 gradients) adds per step.
    allreduce = None
    if world > 1:
        n_params = 24 * (4 * 2048 * 2048 + 2 * 2048 * 8192) + 2 * 65536 * 2048
        grads = torch.zeros(n_params, device=dev, dtype=torch.bfloat16)
        for _ in range(2):
            dist.all_reduce(grads)
        barrier()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record()
        for _ in range(5):
            dist.all_reduce(grads)
        a1.record()
        barrier()
        allreduce = {"ms": a0.elapsed_time(a1) / 5, "bytes": n_params * 2}
        del grads

    # ---- last, because it leaves the GPU at its power cap: the same step back to back for about a second
    sustained = None
    if args.steps >= 10:        # skipped in short runs (launch lists under a profiler)
        s_sampler = ClockSampler(local)
        n_probe = 200
        for i in range(n_probe):
            step(i)
        torch.cuda.synchronize()
        if rank == 0:
            s_sampler.start()
        se = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        n_sus = int(1.2 / 0.000135)
        se[0].record()
        for i in range(n_sus // 3):
            step(i)
        se[1].record()                      # the first third lets power and clocks settle
        for i in range(n_sus - n_sus // 3):
            step(i)
        se[2].record()
        torch.cuda.synchronize()
        s_clocks = s_sampler.stop() if rank == 0 else None
        sus_ms = se[1].elapsed_time(se[2]) / (n_sus - n_sus // 3)
        sustained = {"value": world * FLOP_PER_STEP / (sus_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": sus_ms,
                     "steps": n_sus - n_sus // 3, "clocks": s_clocks}
        _lib.check(lib.pb_gemm_check(stream))

    times = torch.tensor([total_ms, e2e_ms, g_ms, q_ms, big_q_ms, big_qt_ms, big_dq_ms, copy_only_ms, scale["ms"], scale["gemm_ms"],
                          allreduce["ms"] if allreduce else 0.0, big_qt32_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    total_ms, e2e_ms, g_ms, q_ms, big_q_ms, big_qt_ms, big_dq_ms, copy_only_ms, scale_ms, scale_gemm_ms, ar_ms, big_qt32_ms = times.tolist()

    # ---- the end-to-end training step (configs[4]); its own record, not the headline.  It comes last, and after it the ranks only
    # talk through the host group: a rank that failed in it cannot be asked for another GPU collective.
    model_step = None
    if not args.skip_model_step:
        torch.cuda.empty_cache()
        model_step = time_model_step(world, rank, dev, barrier, host_group)
        ms_t = torch.tensor([model_step.get("ms_per_step", -1.0)], dtype=torch.float64)
        bad_t = torch.tensor([0 if "ms_per_step" in model_step else 1], dtype=torch.int32)
        if world > 1:
            dist.all_reduce(ms_t, op=dist.ReduceOp.MAX, group=host_group)
            dist.all_reduce(bad_t, op=dist.ReduceOp.MAX, group=host_group)
        if "ms_per_step" in model_step:
            model_step["ms_per_step"] = ms_t.item()
        if bad_t.item() and "error" not in model_step:
            model_step = {"error": "another rank failed in the end-to-end step"}
        model_failed = bool(bad_t.item())
    else:
        model_failed = False

    if rank == 0:
        peaks = load_peaks()
        ms_per_step = total_ms / args.steps
        fp8_peak = 2.0 * peaks["bf16_tflops"]
        gemm_tflops = FLOP_PER_STEP / (g_ms * 1e-3) / 1e12

        def hbm(kernel, ms, traffic=None):
            gbs = quant_bytes / (ms * 1e-3) / 1e9
            return {"bound": "hbm", "kernel": kernel, "workload": f"X[{qm},{qk}] bf16", "achieved": gbs, "peak": peaks["hbm_gbs"],
                    "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"], "traffic": traffic, "us": ms * 1e3,
                    "peak_source": f"hbm_gbs of {peaks['source']}"}

        so_flop = 6.0 * so_tokens * (4 * so_d * so_d + 2 * so_d * so_ffn)
        out = {
            "metric": METRIC, "value": world * FLOP_PER_STEP / (ms_per_step * 1e-3) / 1e12, "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp8_e4m3 x fp8_e4m3 -> f32",
            "data": "synthetic",
            "config": {"workload": WORKLOAD, "rows_per_gpu": M, "parallelism": f"row shards x{world}, no collective",
                       "l2": f"rotation over {NBUF} buffer sets, {NBUF * (M * K * 3 + M * N * 2) / 1e6:.0f} MB > 126 MB L2",
                       "launch": (f"CUDA graph of {NBUF} steps, replayed" if graph is not None else "eager launches")},
            "gpu_launches": args.steps * 2,      # per step: quantize_row128_bf16_kernel + gemm_tn_pair_kernel
            "parts": {"gemm_ms": g_ms, "gemm_tflops": gemm_tflops, "quantize_ms": q_ms,
                      "quantize_gbs_in_step": M * K * QUANT_BYTES_PER_ELEM / (q_ms * 1e-3) / 1e9,
                      "kernels_per_step": "quantize_row128_bf16 (also lays out the GEMM scales of X), gemm_tn_pair",
                      "how": "per-kernel times come from a second pass over the same steps with a CUDA event after every launch; "
                             "the timed region itself has no events between its launches"},
            "roofline": {"bound": "tensor", "kernel": "gemm_tn_pair_kernel", "achieved": gemm_tflops, "peak": fp8_peak, "unit": "TFLOP/s",
                         "frac": gemm_tflops / fp8_peak, "traffic": GEMM_DRAM_TRAFFIC_BYTES,
                         "peak_source": f"2 x bf16_tflops burst of {peaks['source']} (no FP8 figure is measured); nominal dense FP8 is 4500",
                         "frac_of_nominal_4500": gemm_tflops / 4500.0},
            "roofline_quantize": hbm("quantize_row128_bf16_kernel", big_q_ms, QUANT_DRAM_TRAFFIC_BYTES),
            "roofline_transposed": hbm("transpose_quantize1024_bf16_kernel", big_qt_ms),
            "roofline_dequantize": hbm("dequantize_row128_kernel", big_dq_ms),
            "roofline_transposed_f32": dict(hbm("transpose_quantize1024_f32_ring_kernel", big_qt32_ms), workload=f"X[{qm},{qk}] f32",
                                            achieved=quant32_bytes / (big_qt32_ms * 1e-3) / 1e9,
                                            frac=quant32_bytes / (big_qt32_ms * 1e-3) / 1e9 / peaks["hbm_gbs"]),
            "e2e": {"value": world * FLOP_PER_STEP / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": M * K * 2, "d2h_bytes_per_step": d2h_bytes,
                    "api": "pratchya_b200._nnx_impl.Linear.product (= QArrayImpl(x,(1,128)) @ kernel, the (1,128)-quantized product the "
                           "reference's __matmul__ returns) on a device copy of pinned host X; the product's fp8 bytes and both scale arrays "
                           "copied back to pinned host memory; uploads and downloads on their own streams, two buffer sets",
                    "ms_per_step_runs": e2e_runs, "statistic": "median of 5 passes",
                    "copy_only_ms": copy_only_ms, "frac_of_copy_only": copy_only_ms / e2e_ms,
                    "cpu_affinity": (f"{min(affinity)}-{max(affinity)} ({len(affinity)} CPUs, from nvidia-smi topo -m)" if affinity else None)},
            "scaleout": {"workload": "configs[3]: training triple (fwd+dgrad+wgrad with quantizers) at d_model 4096, FFN 16384, "
                                     f"M = {so_tokens} tokens split by rows over {world} GPU(s), X ~ Student-t(3), weights replicated, no collective",
                         "scaling": "strong", "rows_per_gpu": so_tokens // world, "ms": scale_ms, "gemm_only_ms": scale_gemm_ms,
                         "tflops_aggregate": so_flop / scale_ms / 1e9, "tflops_per_gpu": so_flop / scale_ms / 1e9 / world,
                         "gemm_only_tflops_per_gpu": so_flop / scale_gemm_ms / 1e9 / world,
                         "one_gpu_ms": one_gpu["ms"] if one_gpu else None,
                         "speedup_vs_one_gpu": (one_gpu["ms"] / scale_ms) if one_gpu else None,
                         "timing": "CUDA events, max over ranks; the 1-GPU time is rank 0 running all rows alone in the same process",
                         "per_projection_rank0": scale["per_projection"]},
            "clocks": clocks,
            "clock_note": "the timed region of K steps is shorter than one sampling period unless K is large: the samples bracket it; "
                          "`sustained` carries the clocks seen inside a second-long run of the same step",
        }
        if allreduce is not None:
            bus = allreduce["bytes"] * 2 * (world - 1) / world / (ar_ms * 1e-3) / 1e9
            out["grad_allreduce"] = {"what": "dist.all_reduce (NCCL, sum) of the bf16 gradients of a 24-layer d_model-2048 model with a 65536-token "
                                             "vocabulary: the end-to-end step's only collective (configs[4]); the quantize/GEMM path has none",
                                     "bytes": allreduce["bytes"], "ms": ar_ms, "bus_gbs": bus,
                                     "frac_of_measured_allreduce_725_gbs": bus / 725.0, "timing": "CUDA events, max over ranks, mean of 5"}
        if triple is not None:
            out["triple"] = {"workload": "configs[2]: fwd+dgrad+wgrad of 4x[2048->2048], [2048->8192], [8192->2048] at M = 32768 tokens, dY e4m3",
                             "ms": triple["ms"], "gemm_only_ms": triple["gemm_ms"], "tflops": triple["flop"] / triple["ms"] / 1e9,
                             "gemm_only_tflops": triple["flop"] / triple["gemm_ms"] / 1e9, "per_projection": triple["per_projection"]}
        if model_step is not None:
            if "ms_per_step" in model_step:
                model_step["tokens_per_s"] = world * model_step["tokens_per_gpu"] / (model_step["ms_per_step"] * 1e-3)
            out["model_step"] = dict(model_step, workload=(
                "configs[4]: modified RWKV-7, 24 layers, d_model 2048, head size 64, vocabulary 65536, context 4096, 8 sequences per GPU "
                f"({8 * world} global; the configuration's 64 at 8 GPUs), random token ids, random-init f32 masters; forward + backward (the first "
                "`recomputed_blocks` blocks recomputed in the backward pass, the last `kept_blocks` keep their activations: as many as the "
                "GPU's free memory holds) + bf16 gradient all-reduce (NCCL) + sign-momentum update; every linear layer through linear_fp8, "
                "the WKV-7 scan, the block's element-wise work and the loss, forward and backward, through the package's kernels"),
                scaling="weak", timing="CUDA events around 2 steps after 2 warm-up steps, max over ranks")
        if sustained is not None:
            out["sustained"] = dict(sustained, peak=2.0 * peaks["bf16_tflops_sustained"],
                                    peak_source="2 x bf16_tflops_sustained of " + peaks["source"],
                                    note="the step repeated for about a second (rank 0's own rate x ranks); not the headline value")
        if world == 1:
            out["cpu_baseline"] = cpu_baseline()
        print(json.dumps(out), flush=True)
    if world > 1:
        if model_failed:
            # a rank's GPU work failed: its context cannot take part in the collective teardown of the NCCL group.  Every rank
            # has agreed on that through the host group and has nothing in flight; they leave without another GPU collective.
            sys.stdout.flush()
            sys.stderr.flush()
            os._exit(0)         # the record on rank 0's line carries the error
        dist.destroy_process_group()
    return 0


def run_profile_case(name: str):
    """A few launches of one kernel on a reduced case, for `ncu --set full` captures
    (not a benchmark: prints nothing that is a result)."""
    import torch
    from pratchya_b200._qualia import _ops, quantize_impl, quantize_transposed_impl
    torch.cuda.set_device(0)
    if name == "quantize":
        x = torch.randn(16384, 4096, device="cuda", dtype=torch.bfloat16)      # 134 MB in: larger than L2
        for _ in range(4):
            quantize_impl(x, (1, 128))
    elif name == "transposed":
        x = torch.randn(16384, 4096, device="cuda", dtype=torch.bfloat16)
        for _ in range(4):
            quantize_transposed_impl(x, 128)
    elif name == "activation_f32":
        # the model's f32 activations: the persistent transposed quantizer on f32, and the token-shift lerps as the prologue of
        # both quantizers (six mixes, three of them also token-major), on 4 x 2048 tokens of 4096 channels (134 MB in)
        from pratchya_b200._nnx_impl._glue import token_shift_lerp_quantized
        g = torch.Generator(device="cuda").manual_seed(0)
        x = torch.randn(4, 2048, 4096, device="cuda", generator=g)
        state, mu = torch.randn(4, 1, 4096, device="cuda", generator=g), torch.rand(6, 4096, device="cuda", generator=g)
        for _ in range(3):
            quantize_transposed_impl(x.view(-1, 4096), 128)
            token_shift_lerp_quantized(x, state, mu, (0, 2, 3))
    elif name == "output_cotangent":
        # the first step of a Linear's backward pass: dY [8192, 4096] f32 (134 MB) through the output's dequantize rule into its two
        # fp8 forms, one call; beside it the plain token-major quantizer on the same array
        g = torch.Generator(device="cuda").manual_seed(0)
        y = torch.randn(8192, 4096, device="cuda", generator=g)
        _, y_sc8, y_sc32 = quantize_impl(y, (1, 128))
        dy = torch.randn(8192, 4096, device="cuda", generator=g) * 1e-3
        for _ in range(3):
            _ops.dequantize_bwd_quantize_dual_impl(y_sc8, y_sc32, dy)
            quantize_transposed_impl(dy, 128)
    elif name == "dequantize":
        x = torch.randn(16384, 4096, device="cuda", dtype=torch.bfloat16)
        t = quantize_impl(x, (1, 128))
        for _ in range(4):
            _ops.dequantize_impl(*t, torch.bfloat16, (1, 128))
    elif name == "wkv7":
        from pratchya_b200._nnx_impl import wkv_state_scan
        bsz, steps, heads = 8, 512, 32                      # 6 x 33.5 MB in, 33.5 MB out: larger than L2
        g = torch.Generator(device="cuda").manual_seed(0)
        shape = (bsz, steps, heads * 64)
        decay = torch.exp(-torch.exp(torch.randn(shape, device="cuda", generator=g) * 0.5 - 1.0))
        iclr = torch.sigmoid(torch.randn(shape, device="cuda", generator=g))
        k = torch.randn(shape, device="cuda", generator=g)
        rk = torch.nn.functional.normalize(k.view(bsz, steps, heads, 64), dim=-1).reshape(shape)
        v, r = torch.randn(shape, device="cuda", generator=g), torch.randn(shape, device="cuda", generator=g)
        for _ in range(3):
            wkv_state_scan(None, decay, iclr, rk, k * iclr, v, r, heads)
    elif name == "wkv7_backward":
        from pratchya_b200._nnx_impl import wkv_state_scan
        bsz, steps, heads = 8, 512, 32
        g = torch.Generator(device="cuda").manual_seed(0)
        shape = (bsz, steps, heads * 64)
        decay = torch.exp(-torch.exp(torch.randn(shape, device="cuda", generator=g) * 0.5 - 1.0))
        iclr = torch.sigmoid(torch.randn(shape, device="cuda", generator=g))
        k = torch.randn(shape, device="cuda", generator=g)
        rk = torch.nn.functional.normalize(k.view(bsz, steps, heads, 64), dim=-1).reshape(shape)
        ins = [decay, iclr, rk, k * iclr, torch.randn(shape, device="cuda", generator=g), torch.randn(shape, device="cuda", generator=g)]
        ins = [t.requires_grad_(True) for t in ins]
        dy = torch.randn(shape, device="cuda", generator=g)
        for _ in range(3):
            wkv_state_scan(None, *ins, heads)[1].backward(dy)
    elif name == "glue":
        # the fused element-wise kernels of the RWKV-7 block, forward and backward, on 8 x 1024 tokens of 2048 channels
        # (67 MB per array: the prepare kernels move 14 and 21 of them)
        from pratchya_b200._nnx_impl._glue import rms_norm, token_shift_lerp, wkv_finish, wkv_prepare
        bsz, steps, heads = 8, 1024, 32
        c = heads * 64
        g = torch.Generator(device="cuda").manual_seed(0)
        mk = lambda: torch.randn(bsz, steps, c, device="cuda", generator=g).requires_grad_(True)
        par = lambda *s: torch.randn(*s, device="cuda", generator=g).requires_grad_(True)
        t = torch.arange(steps, device="cuda", dtype=torch.float32)
        freqs = torch.outer(t, 1.0 / (1e4 ** (torch.arange(0, 64, 2, device="cuda", dtype=torch.float32) / 64)))
        cos_tab, sin_tab = torch.cos(freqs), torch.sin(freqs)
        x, state, mu = mk(), par(bsz, 1, c), par(6, c)
        outs = token_shift_lerp(x, state, mu)
        torch.autograd.backward(list(outs), [torch.ones_like(o) for o in outs])
        ins = [mk() for _ in range(7)]
        pre = wkv_prepare(*ins[:5], ins[5], ins[6], cos_tab, sin_tab, par(1, c), par(1, c), heads)
        torch.autograd.backward(list(pre), [torch.ones_like(o) for o in pre])
        fin = wkv_finish(mk(), mk(), mk(), mk(), mk(), par(c), par(c), par(1, c), heads * 1e-5, heads)
        fin.backward(torch.ones_like(fin))
        y = rms_norm(mk(), par(1, c), 1e-6)
        y.backward(torch.ones_like(y))
    elif name == "gemm_full":
        m, n, k = M, N, K                                   # the benchmark's own launch, for DRAM-byte counters only
        x = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(k, n, device="cuda", dtype=torch.bfloat16) * 0.02
        xq, wq = quantize_impl(x, (1, 128)), quantize_impl(w, (128, 128))
        for _ in range(3):
            _ops.matmul_impl(*xq, *wq, (1, 128), (128, 128), out_dtype=torch.bfloat16)
    else:
        m, n, k = 4096, 4096, 2048
        x = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(k, n, device="cuda", dtype=torch.bfloat16) * 0.02
        xq, wq = quantize_impl(x, (1, 128)), quantize_impl(w, (128, 128))
        for _ in range(4):
            _ops.matmul_impl(*xq, *wq, (1, 128), (128, 128), out_dtype=torch.bfloat16)
    torch.cuda.synchronize()
    print(f"profile case {name} done")
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--headline-only", action="store_true",
                    help="only the headline step and its per-kernel pass (for launch lists under a profiler): no e2e, triple, scaleout or CPU leg")
    ap.add_argument("--profile-case", default=None, choices=["gemm", "gemm_full", "quantize", "transposed", "activation_f32", "output_cotangent", "dequantize", "wkv7", "wkv7_backward", "glue"],
                    help="run a few launches of one kernel on a reduced case (for ncu) and exit")
    ap.add_argument("--skip-model-step", action="store_true", help="leave out the end-to-end training-step record (about half a minute)")
    ap.add_argument("--cpu-child", action="store_true", help=argparse.SUPPRESS)
    args = ap.parse_args()
    if args.cpu_child:
        return run_cpu_child(args)
    if args.profile_case:
        return run_profile_case(args.profile_case)
    if args.impl == "reference":
        return run_reference(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
