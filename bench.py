"""Benchmark of the kernel suite (one JSON line on stdout from rank 0).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--headline NAME] [--only NAME[,NAME]] [--no-cpu]

A "step" is one call of the headline workload's hot path on one batch of seeded
synthetic input.  `value` is timed on the device with inputs resident in HBM;
`e2e` times the same call from pinned host buffers (H2D + kernel + D2H).  The
other workloads of the suite are reported under "kernels" (N=1 only).  With
--impl reference the CPU restatement of the reference's own CPU path (numpy
float32, OpenBLAS contractions) is timed on the host cores instead.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "cutile.jl_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

L2_BYTES = 126 * 1024 * 1024


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm=d["hbm_gbs"], tensor=d["bf16_tflops"], tensor_sustained=d["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm=6650.0, tensor=1590.0, tensor_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples the SM clock and the clock-event reasons while the timed regions run (read-only queries).  NVML is
    polled from a thread every 2 ms when the Python binding is there (timed regions of this suite last 5-50 ms);
    otherwise `nvidia-smi -lms 100` is read, the query of the profiling recipe."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.rows = []          # (time, sm_mhz, max_mhz, set of reasons)
        self.proc = None
        self.source = None
        self._stop = threading.Event()

    def start(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = self.gpu
            if vis:
                ids = [v for v in vis.split(",") if v.strip() != ""]
                if self.gpu < len(ids) and ids[self.gpu].strip().isdigit():
                    phys = int(ids[self.gpu])
            h = nv.nvmlDeviceGetHandleByIndex(phys)
            mx = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
            names = (("hw_slowdown", nv.nvmlClocksEventReasonHwSlowdown),
                     ("hw_thermal_slowdown", nv.nvmlClocksEventReasonHwThermalSlowdown),
                     ("sw_thermal_slowdown", nv.nvmlClocksEventReasonSwThermalSlowdown),
                     ("sw_power_cap", nv.nvmlClocksEventReasonSwPowerCap))

            def poll():
                while not self._stop.is_set():
                    try:
                        mhz = float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                        bits = nv.nvmlDeviceGetCurrentClocksEventReasons(h)
                        self.rows.append((time.time(), mhz, mx, {n for n, b in names if bits & b}))
                    except Exception:
                        pass
                    time.sleep(0.002)
            nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)  # raises here if the query is not supported
            self.source = "nvml, 2 ms"
            threading.Thread(target=poll, daemon=True).start()
            return
        except Exception:
            pass
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.gpu), "-lms", "100"], stdout=subprocess.PIPE, text=True)
            self.source = "nvidia-smi, 100 ms"
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            c = [x.strip() for x in line.split(",")]
            if len(c) < 9:
                continue
            try:
                reasons = {n for n, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7),
                                            ("sw_power_cap", 8)) if c[col].lower().startswith("active")}
                self.rows.append((time.time(), float(c[1]), float(c[2]), reasons))
            except ValueError:
                pass

    def stop(self):
        self._stop.set()
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, t0, t1):
        inside = [r for r in self.rows if t0 <= r[0] <= t1]
        rows = inside or [r for r in self.rows if t0 - 0.05 <= r[0] <= t1 + 0.15] or list(self.rows)
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["clock query unavailable"]}
        sm = sorted(r[1] for r in rows)
        reasons = set()
        for r in rows:
            reasons |= r[3]
        return {"sm_mhz": sm[len(sm) // 2], "sm_min_mhz": sm[0], "sm_max_mhz": rows[0][2], "reasons": sorted(reasons),
                "samples": len(rows), "samples_inside_timed_region": len(inside), "source": self.source}


# --------------------------------------------------------------------------- workloads
class Workload:
    """One benchmark configuration.  Subclasses fill in the members below."""
    name = ""
    metric = ""
    unit = ""            # "GB/s" or "TFLOP/s"
    bound = "hbm"        # roofline that binds
    dtype = "f32"
    launches_per_step = 1
    kernel = ""          # name of the dominant kernel
    uses_blas = False    # the CPU baseline's contractions run on all host cores through OpenBLAS

    def work(self):      # algorithmic bytes (hbm) or flops (tensor) per step
        raise NotImplementedError

    def host_inputs(self):  # dict of numpy arrays (seeded)
        raise NotImplementedError

    def to_device(self, host, torch):  # -> state (device tensors incl. outputs)
        raise NotImplementedError

    def step(self, ctb, st):  # enqueue one step on the current stream
        raise NotImplementedError

    def e2e_io(self, st):  # (list of (device, pinned host) input pairs, list of (device, pinned host) outputs)
        raise NotImplementedError

    def cpu_step(self, host, ref, np):  # -> (callable doing one bounded sample, fraction of a step, description)
        raise NotImplementedError

    def check(self, host, st, ref, np):  # parity spot check, returns error figure
        return None


class Softmax(Workload):
    metric = "softmax_gbps"
    unit = "GB/s"
    M = N = 4096

    def __init__(self, variant):
        self.variant = variant
        self.name = "softmax_tma" if variant == 0 else "softmax_chunked"
        self.kernel = "softmax_staged_kernel"

    def describe(self):
        return f"row softmax f32 {self.M}x{self.N} N(0,4) seed 1, variant={'single-tile' if self.variant == 0 else 'chunked-online'}"

    def work(self):
        return 2 * self.M * self.N * 4

    def host_inputs(self):
        from oracle import inputs
        return inputs.softmax(self.M, self.N, seed=1)

    def to_device(self, host, torch):
        x = torch.from_numpy(host["input"]).cuda()
        return dict(x=x, out=torch.empty_like(x))

    def step(self, ctb, st):
        if self.variant == 0:
            ctb.softmax.softmax_tma_kernel(st["out"], st["x"], 4096)
        else:
            ctb.softmax.softmax_chunked_kernel(st["out"], st["x"], self.N, 1024)

    def e2e_io(self, st):
        return [("x",)], [("out",)]

    def cpu_step(self, host, ref, np):
        x = host["input"]
        return (lambda: ref.softmax(x, dtype=np.float32)), 1.0, "full 4096x4096 rows, numpy float32"

    def check(self, host, st, ref, np):
        rows = slice(0, 256)
        return ref.max_abs_over_max(st["out"][rows].cpu().numpy(), ref.softmax(host["input"][rows]))


class LayerNormFwd(Workload):
    name = "layernorm_fwd"
    metric = "layernorm_fwd_gbps"
    unit = "GB/s"
    kernel = "ln_fwd_kernel"
    M = N = 4096

    def describe(self):
        return "LayerNorm fwd f32 4096x4096, X~N(0,1) W~U(.5,1.5) B~N(0,.1) eps 1e-5 seed 0"

    def work(self):
        return 2 * self.M * self.N * 4 + 2 * self.N * 4 + 2 * self.M * 4

    def host_inputs(self):
        from oracle import inputs
        return inputs.layernorm(self.M, self.N, seed=0)

    def to_device(self, host, torch):
        st = {k: torch.from_numpy(host[k]).cuda() for k in ("X", "W", "B", "DY")}
        st.update(Y=torch.empty_like(st["X"]), DX=torch.empty_like(st["X"]),
                  Mean=torch.empty(self.M, device="cuda"), Rstd=torch.empty(self.M, device="cuda"),
                  DWp=torch.empty(64, self.N, device="cuda"), DBp=torch.empty(64, self.N, device="cuda"),
                  FDW=torch.empty(self.N, device="cuda"), FDB=torch.empty(self.N, device="cuda"))
        return st

    def step(self, ctb, st):
        ctb.layernorm.layer_norm_fwd(st["X"], st["W"], st["B"], st["Y"], st["Mean"], st["Rstd"], 1e-5, 1024)

    def e2e_io(self, st):
        return [("X",), ("W",), ("B",)], [("Y",), ("Mean",), ("Rstd",)]

    def cpu_step(self, host, ref, np):
        return (lambda: ref.layernorm_fwd(host["X"], host["W"], host["B"], host["eps"], dtype=np.float32)), 1.0, \
            "full 4096x4096, numpy float32"

    def check(self, host, st, ref, np):
        r = slice(0, 256)
        return ref.max_abs_over_max(st["Y"][r].cpu().numpy(),
                                    ref.layernorm_fwd(host["X"][r], host["W"], host["B"], host["eps"])[0])


class LayerNormBwd(LayerNormFwd):
    name = "layernorm_bwd"
    metric = "layernorm_bwd_gbps"
    kernel = "ln_bwd_kernel"
    launches_per_step = 2

    def describe(self):
        return "LayerNorm bwd f32 4096x4096, dY~N(0,1) seed 0, GROUP_SIZE_M=64 (dX kernel + partial reduce)"

    def work(self):
        return 3 * self.M * self.N * 4 + 3 * self.N * 4 + 2 * self.M * 4

    def to_device(self, host, torch):
        import cutile_b200 as ctb
        st = super().to_device(host, torch)
        LayerNormFwd.step(self, ctb, st)  # Mean/Rstd are inputs of the backward pass
        return st

    def step(self, ctb, st):
        ctb.layernorm.layer_norm_bwd_dx_partial_dwdb(st["DX"], st["DY"], st["DWp"], st["DBp"], st["X"], st["W"],
                                                     st["Mean"], st["Rstd"], None, 64, 1024)
        ctb.layernorm.layer_norm_bwd_dwdb(st["DWp"], st["DBp"], st["FDW"], st["FDB"], 32, 1024)

    def e2e_io(self, st):
        return [("X",), ("DY",), ("W",), ("Mean",), ("Rstd",)], [("DX",), ("FDW",), ("FDB",)]

    def cpu_step(self, host, ref, np):
        y, m, r = ref.layernorm_fwd(host["X"], host["W"], host["B"], host["eps"], dtype=np.float32)
        return (lambda: ref.layernorm_bwd(host["X"], host["W"], host["DY"], m, r, dtype=np.float32)), 1.0, \
            "full 4096x4096, numpy float32"

    def check(self, host, st, ref, np):
        _, m, r = ref.layernorm_fwd(host["X"], host["W"], host["B"], host["eps"])
        dx, dw, db = ref.layernorm_bwd(host["X"], host["W"], host["DY"], m, r)
        return max(ref.max_abs_over_max(st["DX"].cpu().numpy(), dx), ref.max_abs_over_max(st["FDW"].cpu().numpy(), dw),
                   ref.max_abs_over_max(st["FDB"].cpu().numpy(), db))


class Gemm(Workload):
    name = "gemm_tf32"
    metric = "gemm_tf32_tflops"
    unit = "TFLOP/s"
    bound = "tensor"
    peak_scale = 0.5  # TF32 MMAs run at half the bf16 rate the measured peak was taken at
    dtype = "tf32"
    kernel = "gemm_kernel<float>"
    uses_blas = True
    M = N = K = 4096

    def describe(self):
        return "C=A*B f32 (TF32 operands, f32 accumulate) 4096x4096x4096, U(-1,1) seed 2"

    def work(self):
        return 2 * self.M * self.N * self.K

    def host_inputs(self):
        from oracle import inputs
        return inputs.gemm(self.M, self.N, self.K, seed=2)

    def to_device(self, host, torch):
        A, B = torch.from_numpy(host["A"]).cuda(), torch.from_numpy(host["B"]).cuda()
        return dict(A=A, B=B, C=torch.empty(self.N, self.M, device="cuda"))

    def step(self, ctb, st):
        ctb.matmul.matmul_kernel(st["A"], st["B"], st["C"], 64, 64, 64)

    def e2e_io(self, st):
        return [("A",), ("B",)], [("C",)]

    def cpu_step(self, host, ref, np):
        A, B = host["A"], host["B"]
        return (lambda: ref.gemm(A, B, dtype=np.float32)), 1.0, "full 4096^3, numpy float32 matmul (OpenBLAS)"

    def check(self, host, st, ref, np):
        rows = slice(0, 64)  # 64 columns of C (rows of the memory-order array)
        return ref.rel_fro(st["C"][rows].cpu().numpy(), ref.gemm(host["A"], host["B"][rows]))


class BatchedGemm(Gemm):
    name = "bgemm_tf32"
    metric = "batched_gemm_tf32_tflops"
    M, K, N, batch = 1024, 2048, 512, 8

    def describe(self):
        return "batched C=A*B f32/TF32, batch 8 of A[1024x2048]*B[2048x512], U(-1,1) seed 2"

    def work(self):
        return 2 * self.M * self.N * self.K * self.batch

    def host_inputs(self):
        from oracle import inputs
        return inputs.batched_gemm(self.M, self.K, self.N, self.batch, seed=2)

    def to_device(self, host, torch):
        A, B = torch.from_numpy(host["A"]).cuda(), torch.from_numpy(host["B"]).cuda()
        return dict(A=A, B=B, C=torch.empty(self.batch, self.N, self.M, device="cuda"))

    def step(self, ctb, st):
        ctb.batchmatmul.batch_matmul_kernel(st["A"], st["B"], st["C"], 128, 128, 64)

    def cpu_step(self, host, ref, np):
        A, B = host["A"], host["B"]
        return (lambda: ref.batched_gemm(A, B, dtype=np.float32)), 1.0, "full batch 8, numpy float32 matmul (OpenBLAS)"

    def check(self, host, st, ref, np):
        return ref.rel_fro(st["C"][3].cpu().numpy(), ref.gemm(host["A"][3], host["B"][3]))


class Fmha(Workload):
    name = "fmha_causal"
    metric = "fmha_causal_tflops"
    unit = "TFLOP/s"
    bound = "tensor"
    dtype = "f16"
    kernel = "fmha_kernel"
    uses_blas = True
    B, H, S, D = 8, 16, 1024, 64

    def describe(self):
        return ("causal FMHA f16 batch 8 x heads 16 x seq 1024 x dim 64, N(0,1) seed 3, scale 1/8; flops = useful "
                "causal work 4*B*H*D*S*(S+1)/2 (the reference's un-halved count 4*B*H*S*S*D is 2.0x this)")

    def work(self):
        return 4 * self.B * self.H * self.D * self.S * (self.S + 1) // 2

    def host_inputs(self):
        from oracle import inputs
        return inputs.fmha(self.B, self.H, self.S, self.S, self.D, seed=3)

    def to_device(self, host, torch):
        st = {k: torch.from_numpy(host[k]).cuda() for k in ("Q", "K", "V")}
        st["Out"] = torch.empty_like(st["Q"])
        return st

    def step(self, ctb, st):
        # the launch inside cutile_fmha; the output buffer is preallocated for the device-resident timing
        ctb.fmha.fmha_kernel(st["Q"], st["K"], st["V"], st["Out"], 0.125, 0, self.D, self.H, 128, 128, 1, True, True)

    def e2e_io(self, st):
        return [("Q",), ("K",), ("V",)], [("Out",)]

    def cpu_step(self, host, ref, np):
        Q, K, V = host["Q"], host["K"], host["V"]
        return (lambda: ref.fmha(Q, K, V, causal=True, dtype=np.float32)), 1.0, \
            "full batch 8 x 16 heads, numpy float32 (OpenBLAS matmuls)"

    def check(self, host, st, ref, np):
        sl = (slice(7, 8), slice(14, 16))
        want = ref.fmha(host["Q"][sl], host["K"][sl], host["V"][sl], causal=True)
        return ref.rel_fro(st["Out"][sl].cpu().numpy(), want)


class Moe(Workload):
    name = "moe_256"
    metric = "moe_ffn_tflops"
    unit = "TFLOP/s"
    bound = "hbm"
    dtype = "f16"
    kernel = "moe_gemm_kernel"
    uses_blas = True
    launches_per_step = 5  # router, align, gate/up GEMM (+SwiGLU), down GEMM, top-k combine
    T, Hd, E, I, topk = 256, 1024, 32, 2048, 2

    def describe(self):
        return (f"MoE FFN f16 {self.T} tokens x hidden 1024, 32 experts, top-2, SwiGLU inter 2048, seed 4; step = "
                "router + align + gate/up GEMM + down GEMM + combine; flops = 2*T*topk*H*I*3")

    def work(self):
        return 2 * self.T * self.topk * self.Hd * self.I * 3

    def roof_work(self):  # HBM: the expert weights have to stream once
        return self.E * (self.Hd * 2 * self.I + self.I * self.Hd) * 2

    def host_inputs(self):
        from oracle import inputs
        return inputs.moe(self.T, self.Hd, self.E, self.I, self.topk, seed=4)

    def to_device(self, host, torch):
        return {k: torch.from_numpy(host[k]).cuda() for k in ("X", "Wr", "w1", "w2")}

    def step(self, ctb, st):
        w, ids = ctb.moe.moe_router(st["X"], st["Wr"], self.topk)
        st["out"] = ctb.moe.cutile_moe(st["X"], st["w1"], st["w2"], w, ids, 128, 128, 64)

    def e2e_io(self, st):
        return [("X",)], [("out",)]  # the expert weights are model state and stay resident

    def cpu_step(self, host, ref, np):
        def f():
            ids, gates, _ = ref.moe_router(host["X"], host["Wr"], self.topk)
            return ref.moe_ffn(host["X"], host["w1"], host["w2"], gates, ids, dtype=np.float32)
        return f, 1.0, f"full {self.T} tokens, numpy float32 (OpenBLAS matmuls per expert)"

    def check(self, host, st, ref, np):
        ids, gates, _ = ref.moe_router(host["X"], host["Wr"], self.topk)
        sample = np.arange(0, self.T, max(1, self.T // 64))
        want = ref.moe_ffn(host["X"][sample], host["w1"], host["w2"], gates[:, sample], ids[:, sample])
        return ref.rel_fro(st["out"].cpu().numpy()[sample], want)


class Moe4096(Moe):
    name = "moe_4096"
    bound = "tensor"
    T = 4096

    def roof_work(self):
        return self.work()


def registry():
    w = [Fmha(), Moe(), Moe4096(), Gemm(), BatchedGemm(), LayerNormFwd(), LayerNormBwd(), Softmax(0), Softmax(1)]
    return {x.name: x for x in w}


# --------------------------------------------------------------------------- timing
def device_time(torch, dist, fn_steps, steps, warmup, graph=True):
    """`warmup` untimed steps, then exactly `steps` steps between two CUDA events on the launching stream; max over
    ranks.  With graph=True the `steps` launches are captured once into a CUDA graph and the timed region replays
    it, so the figure is device time and not the host's Python launch rate (the reference's protocol brackets single
    launches with events for the same reason, examples/benchmarks.jl:104,159-171)."""
    for i in range(warmup):
        fn_steps(i)
    torch.cuda.synchronize()
    g = None
    if graph:
        g = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            with torch.cuda.graph(g, stream=side):
                for i in range(steps):
                    fn_steps(warmup + i)
        torch.cuda.current_stream().wait_stream(side)
        g.replay()  # one untimed replay: the graph is uploaded before the timed region
        torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.time()
    e0.record()
    if g is not None:
        g.replay()
    else:
        for i in range(steps):
            fn_steps(warmup + i)
    e1.record()
    torch.cuda.synchronize()
    t1 = time.time()
    if dist is not None:
        dist.barrier()
    ms = max_over_ranks(e0.elapsed_time(e1), torch, dist, "cuda")
    return ms, t0, t1


def max_over_ranks(ms, torch, dist, device):
    """The job's time is the slowest rank's (every rank must hold the same figure afterwards)."""
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return float(ms)
    t = torch.tensor([ms], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def aggregate_value(work_per_rank, world, ms_per_step, unit):
    """Whole-job throughput: the units all ranks processed divided by the (max-over-ranks) step time."""
    return work_per_rank * world / (ms_per_step * 1e-3) / (1e9 if unit == "GB/s" else 1e12)


def run_workload(w, torch, ctb, dist, steps, warmup, rank, world, do_e2e, do_cpu, sampler=None):
    import numpy as np
    from oracle import ref
    host = w.host_inputs()
    base = w.to_device(host, torch)
    nbytes = sum(t.numel() * t.element_size() for t in base.values() if hasattr(t, "numel"))
    nsets = max(2, min(8, -(-2 * L2_BYTES // max(nbytes, 1)) + 1))
    sets = [base] + [{k: (v.clone() if hasattr(v, "clone") else v) for k, v in base.items()} for _ in range(nsets - 1)]
    ms, t0, t1 = device_time(torch, dist, lambda i: w.step(ctb, sets[i % nsets]), steps, warmup)
    ctb.check_device_status(torch.cuda.current_device())
    per = ms / steps
    scale = 1e9 if w.unit == "GB/s" else 1e12
    value = aggregate_value(w.work(), world, per, w.unit)
    res = dict(name=w.name, metric=w.metric, unit=w.unit, value=value, ms_per_step=per, work_per_step=w.work(),
               workload=w.describe(), l2="rotating %d input/output sets (%.0f MB total, L2 is 126 MB)" %
               (nsets, nsets * nbytes / 1e6), t0=t0, t1=t1, launches=w.launches_per_step * steps,
               timing="K steps captured in one CUDA graph, replayed between two events")
    res["parity_err"] = w.check(host, sets[(warmup + steps - 1) % nsets], ref, np)
    if do_e2e:
        ins, outs = w.e2e_io(base)
        w.step(ctb, base)  # outputs that the step itself allocates exist from here on
        pin_in = {k[0]: torch.from_numpy(host[k[0]] if k[0] in host else base[k[0]].cpu().numpy()).pin_memory() for k in ins}
        pin_out = {k[0]: torch.empty(base[k[0]].shape, dtype=base[k[0]].dtype).pin_memory() for k in outs}

        def e2e_step(i):
            for k, h in pin_in.items():
                base[k].copy_(h, non_blocking=True)
            w.step(ctb, base)
            for k, h in pin_out.items():
                h.copy_(base[k], non_blocking=True)
        ems, _, _ = device_time(torch, dist, e2e_step, max(3, steps // 4), 3, graph=False)
        eper = ems / max(3, steps // 4)
        res["e2e"] = dict(value=w.work() * world / (eper * 1e-3) / scale, unit=w.unit, ms_per_step=eper,
                          h2d_bytes_per_step=sum(h.numel() * h.element_size() for h in pin_in.values()),
                          d2h_bytes_per_step=sum(h.numel() * h.element_size() for h in pin_out.values()))
    if do_cpu and rank == 0:
        res["cpu_baseline"] = cpu_time(w, host)
    return res


def run_moe_ep(torch, ctb, dist, steps, warmup, rank, world):
    """Expert-parallel MoE at N > 1 (strong scaling): 4096 tokens in total, T/N tokens and 32/N experts per rank,
    router on the local tokens, token rows and expert outputs cross NVLink as stores into peer memory issued by the
    dispatch kernel and by the down projection's epilogue (no all-to-all, no host synchronisation).  Eager
    launches, timed with CUDA events, max over ranks."""
    import numpy as np
    from oracle import inputs
    T, H, E, I, topk = 4096, 1024, 32, 2048, 2
    if E % world or T % world:
        return None
    Tl, El = T // world, E // world
    g = np.random.default_rng(4)
    X = torch.from_numpy(g.standard_normal((T, H), dtype=np.float32).astype(np.float16)[rank * Tl:(rank + 1) * Tl]).cuda()
    Wr = torch.from_numpy((0.02 * g.standard_normal((E, H), dtype=np.float32)).astype(np.float16)).cuda()
    gw = torch.Generator(device="cuda").manual_seed(100 + rank)  # this rank's expert shard, N(0, 0.02)
    w1 = (0.02 * torch.randn(El, 2 * I, H, device="cuda", generator=gw)).half()
    w2 = (0.02 * torch.randn(El, H, I, device="cuda", generator=gw)).half()

    bufs = ctb.moe.EpPeerBuffers(Tl, H, topk, X.device)

    def step(i):
        w, ids = ctb.moe.moe_router(X, Wr, topk)
        return ctb.moe.cutile_moe_ep_peer(bufs, X, w1, w2, w, ids, E, 128, 128, 64)
    ms, _, _ = device_time(torch, dist, step, steps, warmup, graph=True)  # every launch is a kernel of this library
    ctb.check_device_status(torch.cuda.current_device())
    per = ms / steps
    flops = 2 * T * topk * H * I * 3
    return dict(metric="moe_ffn_tflops", value=flops / (per * 1e-3) / 1e12, unit="TFLOP/s", ms_per_step=per,
                scaling="strong", workload=f"expert-parallel MoE f16, {T} tokens in total ({Tl} per rank), {El} of {E} "
                "experts per rank, top-2; step = router + dispatch kernel storing token rows into the owners' peer "
                "memory + barrier kernel + expert FFN whose epilogue stores the outputs into the senders' peer memory "
                "+ barrier kernel + sum over top-k", timing="K steps captured in a CUDA graph per rank and replayed "
                "between two CUDA events, max over ranks")


def cpu_time(w, host, repeats=3):
    import numpy as np
    from oracle import ref
    fn, frac, sample = w.cpu_step(host, ref, np)
    fn()  # warm-up
    best = 1e30
    for _ in range(repeats):
        t = time.perf_counter()
        fn()
        best = min(best, time.perf_counter() - t)
    scale = 1e9 if w.unit == "GB/s" else 1e12
    # numpy's element-wise code is single-threaded; only the OpenBLAS matmuls use every core
    threads = int(os.environ.get("OPENBLAS_NUM_THREADS", os.cpu_count() or 1)) if w.uses_blas else 1
    return dict(value=w.work() * frac / best / scale, unit=w.unit, cores=threads, kind="port",
                sample=sample + f"; best of {repeats}; {best * 1e3:.1f} ms", host_cpus=os.cpu_count())


_RESULT_FD = None


def keep_stdout_for_the_result():
    """File descriptor 1 carries exactly one JSON line.  Libraries write there as well (NCCL prints its version
    banner to stdout while a communicator is set up), so descriptor 1 is pointed at stderr for the rest of the run
    and the result line goes to a private copy of the original."""
    global _RESULT_FD
    if _RESULT_FD is None:
        sys.stdout.flush()
        _RESULT_FD = os.dup(1)
        os.dup2(2, 1)


def emit(line):
    data = (json.dumps(line) + "\n").encode()
    fd = _RESULT_FD if _RESULT_FD is not None else 1
    sys.stdout.flush()
    os.write(fd, data)


def main():
    keep_stdout_for_the_result()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--headline", default=None)
    ap.add_argument("--only", default=None, help="comma-separated workload names (default: all at N=1)")
    ap.add_argument("--no-cpu", action="store_true")
    a = ap.parse_args()
    a.warmup = max(a.warmup, 3)
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    reg = registry()
    headline = a.headline or ("fmha_causal" if "fmha_causal" in reg else "softmax_tma")
    hw = reg[headline]
    pk = peaks()

    if a.impl == "reference":
        if rank != 0:
            return
        host = hw.host_inputs()
        cb = cpu_time(hw, host, repeats=max(1, min(a.steps, 3)))
        line = dict(impl="reference", metric=hw.metric, value=cb["value"], unit=hw.unit, n_gpus=a.gpus, steps=a.steps,
                    warmup=a.warmup, ms_per_step=None, higher_is_better=True, scaling="weak", vs_baseline=None,
                    dtype=hw.dtype, data="synthetic", config={"workload": hw.describe()}, cpu_baseline=cb,
                    e2e=dict(value=cb["value"], unit=hw.unit, h2d_bytes_per_step=0, d2h_bytes_per_step=0),
                    gpu_launches=0,
                    note="CPU restatement of the reference's own CPU check path (numpy float32 + OpenBLAS); the "
                         "reference's GPU path needs Julia and tileiras, which are unavailable on this box")
        emit(line)
        return

    import torch
    import cutile_b200 as ctb  # raises if the CUDA library is missing: there is no fallback
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU path")
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    sampler = ClockSampler(local)
    sampler.start()
    time.sleep(0.3)
    head = run_workload(hw, torch, ctb, dist, a.steps, a.warmup, rank, world, True, not a.no_cpu and world == 1)
    clocks = sampler.summary(head["t0"], head["t1"])
    others = {}
    if world == 1:
        names = [n for n in reg if n != headline]
        if a.only is not None:
            names = [n for n in a.only.split(",") if n in reg and n != headline]  # "--only none": headline alone
        for n in names:
            r = run_workload(reg[n], torch, ctb, None, a.steps, a.warmup, rank, 1, True, not a.no_cpu)
            r["clocks"] = sampler.summary(r["t0"], r["t1"])
            others[n] = r
    if world > 1:
        try:
            ep = run_moe_ep(torch, ctb, dist, max(5, min(a.steps, 30)), 3, rank, world)
        except Exception as e:  # the headline line is still reported; the entry says why it is missing
            sys.stderr.write(f"moe_ep_4096 failed on rank {rank}: {e!r}\n")
            ep = dict(metric="moe_ffn_tflops", unavailable=repr(e)[:300])
        if ep is not None:
            others["moe_ep_4096"] = ep
    sampler.stop()

    # DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of one launch of each workload's dominant kernel,
    # from the ncu captures summarised in profiles/<kernel>_<workload>.txt (for the MoE workloads: gate/up + down
    # launches of moe_gemm_kernel).  Writes are below the algorithmic output bytes wherever the L2 still holds the
    # output when the kernel ends.
    ncu_traffic = {"fmha_causal": 51.35e6, "softmax_tma": 84.48e6, "softmax_chunked": 83.28e6, "layernorm_fwd": 85.46e6,
                   "layernorm_bwd": 170.13e6, "gemm_tf32": 383.89e6, "bgemm_tf32": 104.26e6, "moe_256": 414.27e6,
                   "moe_4096": 483.97e6}

    def roof(r, w):
        peak = pk["hbm"] if w.bound == "hbm" else pk["tensor"] * getattr(w, "peak_scale", 1.0)
        rw = w.roof_work() if hasattr(w, "roof_work") else r["work_per_step"]
        ach = rw / (r["ms_per_step"] * 1e-3) / (1e9 if w.bound == "hbm" else 1e12)
        return dict(bound=w.bound, achieved=ach, peak=peak, unit="GB/s" if w.bound == "hbm" else "TFLOP/s",
                    frac=ach / peak, traffic=ncu_traffic.get(w.name), kernel=w.kernel,
                    peak_source=pk["source"])

    if rank == 0:
        line = dict(metric=hw.metric, value=head["value"], unit=hw.unit, n_gpus=world, steps=a.steps, warmup=a.warmup,
                    ms_per_step=head["ms_per_step"], higher_is_better=True, scaling="weak", vs_baseline=None,
                    dtype=hw.dtype, data="synthetic",
                    config={"workload": hw.describe(), "l2": head["l2"], "per_gpu": "same workload on every rank",
                            "timing": head["timing"]},
                    clocks=clocks, e2e=head.get("e2e"), gpu_launches=head["launches"], roofline=roof(head, hw),
                    cpu_baseline=head.get("cpu_baseline"), parity_err=head["parity_err"])
        if others:
            line["kernels"] = {n: (r if n not in reg else
                                   dict(metric=r["metric"], value=r["value"], unit=r["unit"],
                                        ms_per_step=r["ms_per_step"], roofline=roof(r, reg[n]), e2e=r.get("e2e"),
                                        cpu_baseline=r.get("cpu_baseline"), parity_err=r["parity_err"],
                                        workload=r["workload"], clocks=r["clocks"])) for n, r in others.items()}
        emit(line)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
