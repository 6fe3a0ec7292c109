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
        return ref.max_abs_over_max(st["out"].cpu().numpy(), ref.softmax(host["input"]))


class LayerNormFwd(Workload):
    name = "layernorm_fwd"
    metric = "layernorm_fwd_gbps"
    unit = "GB/s"
    kernel = "ln_fwd_staged_kernel"
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
        return ref.max_abs_over_max(st["Y"].cpu().numpy(), ref.layernorm_fwd(host["X"], host["W"], host["B"], host["eps"])[0])


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
    kernel = "gemm_pair_kernel<float>"
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
        return ("causal FMHA f16 b8 h16 s1024 d64, N(0,1) seed 3, scale 1/8; flops = useful causal work "
                "4*B*H*D*S*(S+1)/2 (the reference counts 4*B*H*S*S*D, 2.0x this)")

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

    def call_surface(self, ctb, st):
        # cutile_fmha allocates Out inside the timed call (examples/fmha.jl:160)
        st["Out"] = ctb.fmha.cutile_fmha(st["Q"], st["K"], st["V"], qk_scale=0.125, causal=True)

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


class SoftmaxOnline(Softmax):
    """Rows too long for one tile of registers (128 KB each): the chunked variant keeps the whole row in shared memory."""
    M, N = 1024, 32768

    def __init__(self):
        Softmax.__init__(self, 1)
        self.name = "softmax_online"
        self.kernel = "softmax_row_smem_kernel"

    def describe(self):
        return f"row softmax f32 {self.M}x{self.N} N(0,4) seed 1, chunked variant, row resident in shared memory (rows longer than one register tile)"

    def step(self, ctb, st):
        ctb.softmax.softmax_chunked_kernel(st["out"], st["x"], self.N, 1024)


class FmhaB64(Fmha):
    """The multi-GPU configuration (batch 64) on one GPU: the T1 of the strong-scaling series."""
    name = "fmha_b64"
    B = 64

    def describe(self):
        return "causal FMHA f16 b64 h16 s1024 d64 (the multi-GPU runs' problem), seed 3; useful causal flops"

    def cpu_step(self, host, ref, np):
        Q, K, V = host["Q"][:8], host["K"][:8], host["V"][:8]
        return (lambda: ref.fmha(Q, K, V, causal=True, dtype=np.float32)), 0.125, "8 of 64 batches, numpy float32"

    def check(self, host, st, ref, np):
        sl = (slice(63, 64), slice(14, 16))
        want = ref.fmha(host["Q"][sl], host["K"][sl], host["V"][sl], causal=True)
        return ref.rel_fro(st["Out"][sl].cpu().numpy(), want)


class VecAdd(Workload):
    name = "vadd"
    metric = "vadd_gbps"
    unit = "GB/s"
    kernel = "vadd_kernel"
    n = 2 ** 27

    def describe(self):
        return "c = a + b, f32, 2^27 elements ~ U(0,1) seed 5 (examples/vadd.jl benchmark shape)"

    def work(self):
        return 3 * self.n * 4

    def host_inputs(self):
        from oracle import inputs
        return inputs.vadd((self.n,), seed=5)

    def to_device(self, host, torch):
        a, b = torch.from_numpy(host["a"]).cuda(), torch.from_numpy(host["b"]).cuda()
        return dict(a=a, b=b, c=torch.empty_like(a))

    def step(self, ctb, st):
        ctb.vadd.vec_add_kernel_1d(st["a"], st["b"], st["c"], 1024)

    def e2e_io(self, st):
        return [("a",), ("b",)], [("c",)]

    def cpu_step(self, host, ref, np):
        a, b = host["a"], host["b"]
        return (lambda: ref.vadd(a, b)), 1.0, "full 2^27 elements, numpy float32"

    def check(self, host, st, ref, np):
        return float(np.max(np.abs(st["c"].cpu().numpy() - ref.vadd(host["a"], host["b"]))))  # exact: 0


class Transpose(Workload):
    name = "transpose"
    metric = "transpose_gbps"
    unit = "GB/s"
    kernel = "transpose_kernel"
    m = n = 8192

    def describe(self):
        return "y = transpose(x), f32 8192x8192 ~ U(0,1) seed 6 (examples/transpose.jl benchmark shape)"

    def work(self):
        return 2 * self.m * self.n * 4

    def host_inputs(self):
        from oracle import inputs
        return inputs.transpose(self.m, self.n, seed=6)

    def to_device(self, host, torch):
        x = torch.from_numpy(host["x"]).cuda()
        return dict(x=x, y=torch.empty(self.m, self.n, device="cuda"))

    def step(self, ctb, st):
        ctb.transpose.transpose_kernel(st["x"], st["y"], 64, 64)

    def e2e_io(self, st):
        return [("x",)], [("y",)]

    def cpu_step(self, host, ref, np):
        x = host["x"]
        return (lambda: ref.transpose(x)), 1.0, "full 8192x8192, numpy float32"

    def check(self, host, st, ref, np):
        return float(np.max(np.abs(st["y"].cpu().numpy() - ref.transpose(host["x"]))))  # exact: 0


class Fft(Workload):
    name = "fft"
    metric = "fft_gbps"
    unit = "GB/s"
    kernel = "fft_kernel"
    batch, factors = 256, (16, 16, 16)

    def describe(self):
        return ("batched complex FFT, 256 x 4096 points as (16, 16, 16) DFT-matrix stages, c64 ~ N(0,1) seed 7 "
                "(examples/fft.jl benchmark shape; the example reports the time, ms_per_step here)")

    def work(self):
        return 2 * self.batch * 4096 * 8

    def host_inputs(self):
        from oracle import inputs
        return inputs.fft(self.batch, self.factors, seed=7)

    def to_device(self, host, torch):
        import cutile_b200 as ctb
        x = torch.from_numpy(host["input"]).cuda()
        return dict(x=x, y=torch.empty_like(x), plan=ctb.fft.FftPlan(self.factors, "cuda"))

    def step(self, ctb, st):
        st["plan"](st["x"], st["y"])

    def e2e_io(self, st):
        return [("x",)], [("y",)]

    def cpu_step(self, host, ref, np):
        x = host["input"][:64]
        tabs = ref.fft_make_twiddles(self.factors)
        return (lambda: ref.fft_three_stage(x, *tabs, self.factors, dtype=np.float32)), 64 / self.batch, \
            "64 of 256 batch items, numpy complex64 three-stage restatement"

    def check(self, host, st, ref, np):
        y = st["y"].cpu().numpy()
        want = ref.fft(host["input"])
        return ref.rel_fro(np.stack([y.real, y.imag]), np.stack([want.real, want.imag]))


class TiledFused(Workload):
    name = "tiled_fused"
    metric = "tiled_broadcast_gbps"
    unit = "GB/s"
    kernel = "tiled_broadcast_pipe_kernel"
    n = 1 << 26

    def describe(self):
        return "ct.Tiled(C) .= A .+ A .* sin.(A) as one kernel, f32, 2^26 elements ~ U(-1,1) seed 8 (test/host/broadcast.jl:13-19)"

    def work(self):
        return 2 * self.n * 4

    def host_inputs(self):
        import numpy as np
        g = np.random.default_rng(8)
        return dict(a=(g.random(self.n, dtype=np.float32) * 2 - 1))

    def to_device(self, host, torch):
        a = torch.from_numpy(host["a"]).cuda()
        return dict(a=a, c=torch.empty_like(a))

    def step(self, ctb, st):
        T = ctb.tiled
        A = T.Tiled(st["a"])
        T.assign(st["c"], A + A * T.sin(A))

    def e2e_io(self, st):
        return [("a",)], [("c",)]

    def cpu_step(self, host, ref, np):
        a = host["a"][: 1 << 22]
        return (lambda: ref.tiled_broadcast(("add", a, ("mul", a, ("sin", a))), dtype=np.float32)), (1 << 22) / self.n, \
            "2^22 of 2^26 elements, numpy float32"

    def check(self, host, st, ref, np):
        a = host["a"][: 1 << 20]
        want = ref.tiled_broadcast(("add", a, ("mul", a, ("sin", a))))
        return float(np.max(np.abs(st["c"][: 1 << 20].cpu().numpy() - want)))


class TiledSum(Workload):
    name = "tiled_sum"
    metric = "tiled_mapreduce_gbps"
    unit = "GB/s"
    kernel = "tiled_reduce_kernel"
    m = n = 8192

    def describe(self):
        return "sum(ct.Tiled(A); dims=1), f32 8192x8192 ~ U(0,1) seed 9 (test/host/mapreduce.jl:16-21)"

    def work(self):
        return self.m * self.n * 4 + self.n * 4

    def host_inputs(self):
        import numpy as np
        return dict(a=np.random.default_rng(9).random((self.n, self.m), dtype=np.float32))

    def to_device(self, host, torch):
        return dict(a=torch.from_numpy(host["a"]).cuda(), out=torch.empty(self.n, 1, device="cuda"))

    def step(self, ctb, st):
        ctb.tiled.tsum(ctb.tiled.Tiled(st["a"]), dims=1, out=st["out"])

    def e2e_io(self, st):
        return [("a",)], [("out",)]

    def cpu_step(self, host, ref, np):
        a = host["a"]
        return (lambda: ref.tiled_mapreduce("identity", "add", a, (1,), dtype=np.float32)), 1.0, "full 8192x8192, numpy float32"

    def check(self, host, st, ref, np):
        want = ref.tiled_mapreduce("identity", "add", host["a"], (1,))
        return ref.rel_fro(st["out"].cpu().numpy(), want)


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

    def call_surface(self, ctb, st):
        # cutile_moe from routing ids to the result, allocating its output (examples/moe.jl:218-257)
        if "w" not in st:
            st["w"], st["ids"] = ctb.moe.moe_router(st["X"], st["Wr"], self.topk)
        st["out"] = ctb.moe.cutile_moe(st["X"], st["w1"], st["w2"], st["w"], st["ids"], 128, 128, 64)

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
    w = [Fmha(), FmhaB64(), Moe(), Moe4096(), Gemm(), BatchedGemm(), LayerNormFwd(), LayerNormBwd(), Softmax(0), Softmax(1),
         SoftmaxOnline(), VecAdd(), Transpose(), Fft(), TiledFused(), TiledSum()]
    return {x.name: x for x in w}


# --------------------------------------------------------------------------- timing
def time_graph(torch, dist, fn_steps, steps, warmup, target_s=0.1, max_replays=400, graph=True):
    """`warmup` untimed steps, then R timed regions of exactly `steps` steps each, every region between its own pair
    of CUDA events on the launching stream, a barrier + synchronize before the first and after the last; the job's
    time is the maximum over ranks.  With graph=True the `steps` launches are captured once into a CUDA graph and each
    region replays it, so the figure is device time and not the host's Python launch rate (the reference's protocol
    brackets single launches with events for the same reason, examples/benchmarks.jl:104,159-171).  R is chosen so that
    the regions together last about `target_s`: long enough for the clock samples (every 2 ms) to fall inside."""
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

    def region():
        if g is not None:
            g.replay()
        else:
            for i in range(steps):
                fn_steps(warmup + i)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(); region(); e1.record()       # one untimed region: the graph is uploaded, and it sizes R
    torch.cuda.synchronize()
    first = max(e0.elapsed_time(e1), 1e-3)
    replays = int(max(3, min(max_replays, target_s * 1e3 / first)))
    if dist is not None:
        t = torch.tensor([replays], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)  # every rank times the same number of regions
        replays = int(t.item())
        dist.barrier()
    torch.cuda.synchronize()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(replays)]
    t0 = time.time()
    for a, b in evs:
        a.record(); region(); b.record()
    torch.cuda.synchronize()
    t1 = time.time()
    if dist is not None:
        dist.barrier()
    per = [a.elapsed_time(b) / steps for a, b in evs]
    mean = max_over_ranks(sum(per) / len(per), torch, dist, "cuda")
    best = max_over_ranks(min(per), torch, dist, "cuda")
    return dict(ms=mean, min_ms=best, max_ms=max(per), replays=replays, t0=t0, t1=t1)


def protocol_times(torch, fn, warm=5, iters=20):
    """The reference's own measurement protocol (examples/benchmarks.jl:104,159-171): 5 warm-up calls, then 20 calls each
    between its own pair of CUDA events; returns (min, mean) in ms.  Single eager calls: the host's launch cost and the
    gaps between a call's kernels are part of the figure, as they are in the reference's."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); fn(); b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    return min(ts), sum(ts) / len(ts)


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


def shard_range(total, world, rank):
    """[lo, hi) of `total` independent units (batches, tokens, experts) on `rank`: contiguous, sizes differ by at most
    one, earlier ranks take the larger shards."""
    base, extra = divmod(total, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def profile_traffic(workload):
    """DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of one launch of every kernel captured in
    profiles/*_<workload>.txt (the ncu summaries of this repository), or None when there is no such file."""
    import glob
    import re
    files = glob.glob(os.path.join(ROOT, "profiles", f"*_{workload}.txt"))
    if not files:
        return None
    scale = {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9}
    per_kernel = {}
    cur = None
    for line in open(files[0]):
        if line.startswith("== "):
            name = line[3:].split("  grid")[0].strip()
            cur = name if name not in per_kernel else None  # the first launch of each kernel
            if cur:
                per_kernel[cur] = 0.0
        elif cur:
            m = re.match(r"\s+dram__bytes_(read|write)\.sum \[(\w+)\] = ([\d.,]+)", line)
            if m:
                per_kernel[cur] += float(m.group(3).replace(",", "")) * scale.get(m.group(2), 1.0)
    tot = sum(per_kernel.values())
    return tot if tot > 0 else None


def e2e_pipelined(torch, w, ctb, host, base, steps):
    """The public call from pinned host buffers, as a three-stage pipeline over two sets of device buffers: the
    host-to-device copies of step i+1 (copy stream), the kernels of step i (compute stream) and the device-to-host
    copy of step i-1's result (second copy stream) overlap.  Every step moves its inputs in and its result out;
    returns (ms per step, bytes in, bytes out)."""
    ins, outs = w.e2e_io(base)
    w.step(ctb, base)  # outputs that the step itself allocates exist from here on
    torch.cuda.synchronize()
    sets = [base, {k: (v.clone() if hasattr(v, "clone") else v) for k, v in base.items()}]
    pin_in = {k[0]: torch.from_numpy(host[k[0]] if k[0] in host else base[k[0]].cpu().numpy()).pin_memory() for k in ins}
    pin_out = [{k[0]: torch.empty(base[k[0]].shape, dtype=base[k[0]].dtype).pin_memory() for k in outs} for _ in range(2)]
    cs, up, down = torch.cuda.current_stream(), torch.cuda.Stream(), torch.cuda.Stream()
    done_k = [None, None]   # kernel of the step that last used buffer set b
    done_d = [None, None]   # its result has left the device

    def run(n):
        for i in range(n):
            b = i & 1
            st = sets[b]
            with torch.cuda.stream(up):
                if done_k[b] is not None:
                    up.wait_event(done_k[b])      # the inputs of set b are free again
                for k, h in pin_in.items():
                    st[k].copy_(h, non_blocking=True)
                ready = torch.cuda.Event(); ready.record(up)
            cs.wait_event(ready)
            if done_d[b] is not None:
                cs.wait_event(done_d[b])          # the previous result of set b has been copied out
            w.step(ctb, st)
            done_k[b] = torch.cuda.Event(); done_k[b].record(cs)
            with torch.cuda.stream(down):
                down.wait_event(done_k[b])
                for k, h in pin_out[b].items():
                    h.copy_(st[k], non_blocking=True)
                done_d[b] = torch.cuda.Event(); done_d[b].record(down)
        cs.wait_stream(up)
        cs.wait_stream(down)
    run(3)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record(cs); run(steps); b.record(cs)
    torch.cuda.synchronize()
    return (a.elapsed_time(b) / steps, sum(h.numel() * h.element_size() for h in pin_in.values()),
            sum(h.numel() * h.element_size() for h in pin_out[0].values()))


def run_workload(w, torch, ctb, dist, steps, warmup, rank, world, do_e2e, do_cpu, target_s=0.1):
    """Times one workload (for the batch-sharded runs: this rank's share of it) on this rank's device."""
    import numpy as np
    from oracle import ref
    host = w.host_inputs()
    base = w.to_device(host, torch)
    nbytes = sum(t.numel() * t.element_size() for t in base.values() if hasattr(t, "numel"))
    nsets = max(2, min(8, -(-2 * L2_BYTES // max(nbytes, 1)) + 1))
    sets = [base] + [{k: (v.clone() if hasattr(v, "clone") else v) for k, v in base.items()} for _ in range(nsets - 1)]
    tm = time_graph(torch, dist, lambda i: w.step(ctb, sets[i % nsets]), steps, warmup, target_s)
    ctb.check_device_status(torch.cuda.current_device())
    res = dict(name=w.name, metric=w.metric, unit=w.unit, ms_per_step=tm["ms"], min_ms=tm["min_ms"], replays=tm["replays"],
               work_per_step=w.work(), t0=tm["t0"], t1=tm["t1"], launches=w.launches_per_step * steps * tm["replays"],
               l2="%d rotating input/output sets, %.0f MB" % (nsets, nsets * nbytes / 1e6))
    res["parity_err"] = w.check(host, sets[(warmup + steps - 1) % nsets], ref, np)
    # the reference's protocol: single eager calls, kernel-only (outputs preallocated) and call surface (the wrapper
    # that allocates its result, where the reference has one)
    res["protocol"] = dict(zip(("min_ms", "mean_ms"), protocol_times(torch, lambda: w.step(ctb, base))))
    if hasattr(w, "call_surface"):
        res["protocol"].update(zip(("call_min_ms", "call_mean_ms"), protocol_times(torch, lambda: w.call_surface(ctb, base))))
    if do_e2e:
        ems, bi, bo = e2e_pipelined(torch, w, ctb, host, base, max(4, min(12, steps // 2)))
        ems = max_over_ranks(ems, torch, dist, "cuda")
        res["e2e"] = dict(ms_per_step=ems, h2d_bytes_per_step=bi, d2h_bytes_per_step=bo)
    if do_cpu and rank == 0:
        res["cpu_baseline"] = cpu_time(w, host)
    return res


def run_moe_ep(torch, ctb, dist, steps, warmup, rank, world, local):
    """Expert-parallel MoE at N > 1 (strong scaling): BASELINE's 4096 tokens in total, 4096/N tokens and 32/N experts
    per rank, through the library's C entry point (ctb_moe_ffn_ep) in both exchange modes.  Checked against the
    single-GPU cutile_moe on the gathered problem (bit for bit, every rank, outside the timed regions) and, for 256
    tokens, against the float64 oracle."""
    import numpy as np
    from oracle import inputs, ref
    T, H, E, I, topk = 4096, 1024, 32, 2048, 2
    if E % world or T % world:
        return None
    Tl, El = T // world, E // world
    d = inputs.moe(tokens=T, hidden=H, experts=E, inter=I, topk=topk, seed=4)  # the same arrays on every rank
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    my, mine = slice(rank * Tl, (rank + 1) * Tl), slice(rank * El, (rank + 1) * El)
    X, Wr = dev(d["X"][my]), dev(d["Wr"])
    w1, w2 = dev(d["w1"][mine]), dev(d["w2"][mine])
    ep = ctb.multi.EpRank(Tl, H, topk, torch.device("cuda", local))
    ctb.multi.reserve_workspace(local, max(ctb.multi.workspace_bytes("moe_ep", Tl, H, I, El, topk, 128, world),
                                           ctb.multi.workspace_bytes("moe_ffn", T, H, I, E, topk, 128)))
    # ---- correctness at the measured configuration
    Xf, w1f, w2f = dev(d["X"]), dev(d["w1"]), dev(d["w2"])
    gf, idf = ctb.moe.moe_router(Xf, Wr, topk)
    full = ctb.moe.cutile_moe(Xf, w1f, w2f, gf, idf, 128, 128, 64)
    g, ids = ctb.moe.moe_router(X, Wr, topk)
    same = {}
    for mode in ("peer", "nccl"):
        out = ep.cutile_moe_ep(X, w1, w2, g, ids, E, 128, 128, 64, a2a_mode=mode)
        torch.cuda.synchronize()
        t = torch.tensor([1 if torch.equal(out, full[my]) else 0], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        same[mode] = bool(t.item())
    sample = np.arange(0, T, T // 256)
    rid, rg, _ = ref.moe_router(d["X"][sample], d["Wr"], topk)
    perr = ref.rel_fro(full.cpu().numpy()[sample], ref.moe_ffn(d["X"][sample], d["w1"], d["w2"], rg, rid)) if rank == 0 else None
    del Xf, w1f, w2f, full
    torch.cuda.empty_cache()
    # ---- timing.  The expert shard is rotated through enough copies to exceed twice the L2 (the 1-GPU moe_4096
    # row streams its weights from HBM as well).
    shard_bytes = (w1.numel() + w2.numel()) * 2
    nsets = max(2, -(-2 * L2_BYTES // shard_bytes) + 1)
    wsets = [(w1, w2)] + [(w1.clone(), w2.clone()) for _ in range(nsets - 1)]
    outs = torch.empty((Tl, H), dtype=torch.float16, device="cuda")

    def step(mode):
        def f(i):
            a, b = wsets[i % nsets]
            gg, ii = ctb.moe.moe_router(X, Wr, topk)
            ep.cutile_moe_ep(X, a, b, gg, ii, E, 128, 128, 64, a2a_mode=mode, out=outs)
        return f
    flops = 2 * T * topk * H * I * 3
    res = dict(metric="moe_ffn_tflops", u="TFLOP/s", bit_identical=same, err=perr, scaling="strong",
               workload=f"{T} tokens, top-2, {El} of {E} experts and {Tl} tokens per rank, seed 4",
               l2=f"{nsets} rotating copies of the expert shard ({nsets * shard_bytes / 1e6:.0f} MB per rank)")
    tp = time_graph(torch, dist, step("peer"), steps, warmup, 0.05)  # kernel launches only: captured in a graph
    ctb.check_device_status(local)
    res.update(v=flops / (tp["ms"] * 1e-3) / 1e12, ms=tp["ms"], min_ms=tp["min_ms"], replays=tp["replays"])
    tn = time_graph(torch, dist, step("nccl"), max(3, steps // 4), 2, 0.02, graph=False)  # reads counts on the host
    ctb.check_device_status(local)
    res["nccl"] = dict(v=flops / (tn["ms"] * 1e-3) / 1e12, ms=tn["ms"])
    ep.close()
    return res


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
    return dict(value=r4(w.work() * frac / best / scale), unit=w.unit, cores=threads, kind="port",
                sample=sample + f"; best of {repeats}; {best * 1e3:.1f} ms", host_cpus=os.cpu_count())


def comparators(torch, pk):
    """Library kernels on the same box, for orientation only (never on the measured path): cuBLAS TF32 GEMM, whose rate
    serves as the TF32 tensor peak of the GEMM rooflines, and torch's scaled_dot_product_attention on the FMHA shapes."""
    out = {}
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        n = 8192
        a, b = torch.randn(n, n, device="cuda"), torch.randn(n, n, device="cuda")
        best = min(protocol_times(torch, lambda: torch.matmul(a, b), 3, 10)[0], 1e9)
        out["cublas_tf32_8192_tflops"] = 2 * n ** 3 / (best * 1e-3) / 1e12
        del a, b
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old
    import torch.nn.functional as F
    for bsz in (8, 64):
        g = torch.Generator(device="cuda").manual_seed(3)
        sets = [[torch.randn(bsz, 16, 1024, 64, device="cuda", generator=g).half() for _ in range(3)]
                for _ in range(4 if bsz == 8 else 2)]
        tm = time_graph(torch, None, lambda i: F.scaled_dot_product_attention(*sets[i % len(sets)], is_causal=True, scale=0.125),
                        10, 3, 0.05)
        out[f"sdpa_b{bsz}_tflops"] = 4 * bsz * 16 * 64 * 1024 * 1025 // 2 / (tm["ms"] * 1e-3) / 1e12
        del sets
    torch.cuda.empty_cache()
    return out


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


def r4(x):
    """Four significant digits: the line has to stay short enough to be kept whole by whoever records it."""
    return None if x is None else float(f"{x:.4g}")


def main():
    keep_stdout_for_the_result()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--headline", default=None)
    ap.add_argument("--only", default=None, help="comma-separated workload names (default: all at N=1)")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-compare", action="store_true", help="skip the library comparators (cuBLAS TF32, torch SDPA)")
    a = ap.parse_args()
    a.warmup = max(a.warmup, 3)
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    reg = registry()
    headline = a.headline or "fmha_causal"
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
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")  # plain peer stores and ring/tree NCCL: no multicast objects
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    sampler = ClockSampler(local)
    sampler.start()
    time.sleep(0.2)
    scale = lambda u: 1e9 if u == "GB/s" else 1e12

    # ---- headline.  N = 1: BASELINE's single-GPU configuration (batch 8).  N > 1: its multi-GPU configuration, batch 64
    # sharded by batch over the ranks with no data-path collective (strong scaling: the total work is fixed).
    sharded = world > 1 and headline == "fmha_causal"
    if sharded:
        hw = reg["fmha_b64"]
        lo, hi = shard_range(hw.B, world, rank)
        head = run_workload(ShardedFmha(hw, lo, hi), torch, ctb, dist, a.steps, a.warmup, rank, world, True, False, 0.25)
        head["work_total"] = hw.work()
    else:
        head = run_workload(hw, torch, ctb, dist, a.steps, a.warmup, rank, world, True, not a.no_cpu and world == 1, 0.25)
        head["work_total"] = hw.work() * world
    clocks = sampler.summary(head["t0"], head["t1"])
    tf32_peak = None
    comp = {}
    if rank == 0 and world == 1 and not a.no_compare:
        comp = comparators(torch, pk)
        tf32_peak = comp.get("cublas_tf32_8192_tflops")

    def peak_of(w):
        if w.bound == "hbm":
            return pk["hbm"], "GB/s"
        if getattr(w, "peak_scale", 1.0) != 1.0:  # TF32: the cuBLAS TF32 rate measured in this run, else half the bf16 figure
            return (tf32_peak or pk["tensor"] * w.peak_scale), "TFLOP/s"
        return pk["tensor"], "TFLOP/s"

    def roof(r, w, work=None):
        peak, unit = peak_of(w)
        rw = work if work is not None else (w.roof_work() if hasattr(w, "roof_work") else r["work_per_step"])
        ach = rw / (r["ms_per_step"] * 1e-3) / scale(unit)
        return dict(bound=w.bound, achieved=r4(ach), peak=r4(peak), unit=unit, frac=r4(ach / peak),
                    traffic=profile_traffic(w.name), kernel=w.kernel, peak_source=pk["source"])

    kernels = {}
    kernel_mhz = []  # median SM clock inside each workload's timed region
    if world == 1:
        names = [n for n in reg if n != headline]
        if a.only is not None:
            names = [n for n in a.only.split(",") if n in reg and n != headline]  # "--only none": headline alone
        for n in names:
            w = reg[n]
            r = run_workload(w, torch, ctb, None, a.steps, a.warmup, rank, 1, True, not a.no_cpu, 0.1)
            ck = sampler.summary(r["t0"], r["t1"])
            rf = roof(r, w)
            # one row per workload, columns named in kernels["cols"]: v value [GB/s for hbm-bound, TFLOP/s for
            # tensor-bound], ms mean per step, frac of the binding roofline b (h = HBM, t = tensor), traf DRAM MB per step
            # from the ncu summary, e2e ms per step from pinned host memory, p1 min ms of the reference's protocol
            # (5 warm-up, 20 single calls), cpu baseline in the value's unit, err parity figure
            traf = None if rf["traffic"] is None else round(rf["traffic"] / 1e6, 1)
            kernels[n] = [r4(w.work() / (r["ms_per_step"] * 1e-3) / scale(w.unit)), r4(r["ms_per_step"]), rf["frac"],
                          rf["bound"][0], traf, r4(r["e2e"]["ms_per_step"]), r4(r["protocol"]["min_ms"]),
                          r4((r.get("cpu_baseline") or {}).get("value")), r4(r["parity_err"])]
            if ck.get("sm_mhz"):
                kernel_mhz.append(ck["sm_mhz"])
        if kernels:
            kernels = dict(cols="v ms frac b traf_MB e2e_ms p1_ms cpu err", **kernels)
    else:
        # batched GEMM sharded by batch (strong scaling, no collective)
        bw = reg["bgemm_tf32"]
        lo, hi = shard_range(bw.batch, world, rank)
        r = run_workload(ShardedBgemm(bw, lo, hi), torch, ctb, dist, a.steps, a.warmup, rank, world, False, False, 0.05)
        if True:
            kernels["bgemm_tf32_sharded"] = dict(v=r4(bw.work() / (r["ms_per_step"] * 1e-3) / 1e12), u="TFLOP/s", ms=r4(r["ms_per_step"]),
                                                 min_ms=r4(r["min_ms"]), scaling="strong",
                                                 workload=f"batch 8 of A[1024x2048]*B[2048x512] TF32 split by batch over {world} ranks, "
                                                          "no collective")
        try:
            ep = run_moe_ep(torch, ctb, dist, max(5, min(a.steps, 20)), 3, rank, world, local)
        except Exception as e:  # the headline line is still reported; the entry says why it is missing
            sys.stderr.write(f"moe_ep_4096 failed on rank {rank}: {e!r}\n")
            ep = dict(metric="moe_ffn_tflops", unavailable=repr(e)[:300])
        if ep is not None:
            for k in ("v", "ms", "min_ms", "err"):
                if k in ep:
                    ep[k] = r4(ep[k])
            kernels["moe_ep_4096"] = ep
    sampler.stop()

    if rank == 0:
        per = head["ms_per_step"]
        value = head["work_total"] / (per * 1e-3) / scale(hw.unit)
        e2e = head.get("e2e")
        if e2e:
            e2e = dict(value=r4(head["work_total"] / (e2e["ms_per_step"] * 1e-3) / scale(hw.unit)), unit=hw.unit,
                       ms_per_step=r4(e2e["ms_per_step"]), h2d_bytes_per_step=e2e["h2d_bytes_per_step"],
                       d2h_bytes_per_step=e2e["d2h_bytes_per_step"], how="pinned host; H2D | kernels | D2H on 3 streams")
        cfg = {"workload": hw.describe(), "l2": head["l2"], "replays": head["replays"],
               "timing": "K-step CUDA graph, R replays each between CUDA events, mean, max over ranks",
               "per_gpu": (f"batch {hw.B // world} of 64 per rank, sharded by batch, no collective" if sharded
                           else "the whole workload on one GPU")}
        line = dict(metric=hw.metric, value=r4(value), unit=hw.unit, n_gpus=world, steps=a.steps, warmup=a.warmup,
                    ms_per_step=r4(per), min_ms_per_step=r4(head["min_ms"]), higher_is_better=True,
                    scaling="strong" if sharded else "weak", vs_baseline=None, dtype=hw.dtype, data="synthetic", config=cfg,
                    clocks=clocks, e2e=e2e, gpu_launches=head["launches"],
                    roofline=roof(head, hw, work=head["work_per_step"] if sharded else None), cpu_baseline=head.get("cpu_baseline"),
                    parity_err=r4(head["parity_err"]),
                    protocol=dict({k: r4(v) for k, v in head["protocol"].items()},
                                  how="5 warm-up, 20 single calls; call_* = allocating wrapper"))
        if comp:  # library kernels on the same box, for orientation (cuBLAS TF32 is the TF32 peak of the GEMM rows)
            line["comparators"] = {k: r4(v) for k, v in comp.items()}
        if kernel_mhz:
            line["clocks"]["kernels_sm_mhz_min"] = min(kernel_mhz)
        if kernels:
            line["kernels"] = kernels
        emit(line)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


class ShardedFmha(FmhaB64):
    """Batches [lo, hi) of the batch-64 FMHA problem: one rank's share when the batch * head items are split by batch
    (the (D, S, H, B) arrays are batch-last, so a share is a contiguous slab)."""

    def __init__(self, whole, lo, hi):
        self.lo, self.hi, self.B = lo, hi, hi - lo

    def host_inputs(self):
        d = FmhaB64().host_inputs()
        return {k: (v[self.lo:self.hi] if k in ("Q", "K", "V") else v) for k, v in d.items()}

    def check(self, host, st, ref, np):
        sl = (slice(self.B - 1, self.B), slice(14, 16))
        want = ref.fmha(host["Q"][sl], host["K"][sl], host["V"][sl], causal=True)
        return ref.rel_fro(st["Out"][sl].cpu().numpy(), want)


class ShardedBgemm(BatchedGemm):
    """Batches [lo, hi) of the batch-8 GEMM problem (batch-last arrays: a contiguous slab per rank)."""

    def __init__(self, whole, lo, hi):
        self.lo, self.hi, self.batch = lo, hi, hi - lo

    def host_inputs(self):
        d = BatchedGemm().host_inputs()
        return {k: (v[self.lo:self.hi] if k in ("A", "B") else v) for k, v in d.items()}

    def check(self, host, st, ref, np):
        return ref.rel_fro(st["C"][0].cpu().numpy(), ref.gemm(host["A"][0], host["B"][0]))


if __name__ == "__main__":
    main()
