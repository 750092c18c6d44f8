"""Benchmark of the SD3.5-medium MMDiT-X denoiser forward on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Metric: denoise steps/s at 1024x1024, batch 8, bf16 (one step = one full
denoiser forward for a batch of 8 samples: latent 16x128x128 -> 4096 image
tokens, 333 context tokens x 4096, pooled 2048, 24 blocks, first 13 with the
extra image-only attention).  Weights are random N(0, 0.02) of the SD3.5-medium
architecture and inputs are N(0, 1) (seed 2): synthetic stand-ins, no dataset
or checkpoint is involved.

With N ranks the batch of 8 is SPLIT across the GPUs (8/N samples each, every
GPU holds the full weight set, no collective on the data path): `value` is
batch-8 steps per second, timed with CUDA events, MAX over ranks ("strong"
scaling).  `weak_value` is the older figure, every rank running a whole batch
of 8.  Extra keys on the same JSON line, printed by rank 0: `c5` (one
2048x2048 image, token-sharded over the N GPUs with an all-to-all around each
attention, checked against the one-GPU forward in the same run), `c4` (the
28-step sampling loop with classifier-free guidance, 16 images over the N
GPUs, bf16 and FP8), `kernels` (per-kernel roofline table with library
attention kernels as context rows).

--impl reference times the reference's CPU implementation of the same path on
the host cores: its own PyTorch modules when a checkout of the reference sits
next to this repository (or SD3_REFERENCE_ROOT points to one), else their
restatement in oracle/mmdit_oracle.py.  One real batch-8 forward is timed once;
each of the K timed steps is one of the eight samples of a step.
"""
import argparse
import importlib.util
import json
import os
import statistics
import subprocess
import sys
import threading
import time

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)

METRIC = "SD3.5-M DiT denoise steps/sec @1024^2 b8 bf16"
WORKLOAD = ("SD3.5-medium DiT forward, 1024^2, batch 8, bf16, 4096 image + 333 context tokens, "
            "24 blocks (13 dual)")
UNIT = "steps/s"
# algorithmic FLOPs of one step (2MNK per GEMM + 4 T^2 E per attention), batch 8
STEP_TFLOP = 89.997
B, TC, HW, TX = 8, 333, 128, 4096
E, NH, FH = 1536, 24, 6144
T = TC + TX
# DRAM bytes (read + written) of one joint-attention launch per sample, from the ncu
# capture of `--profile-case attn_joint` (batch 2: 81.74 MB read + 7.83 MB written);
# it is the compulsory q|k|v read and O write, so it grows in proportion to the batch.
ATTN_TRAFFIC_BYTES_PER_SAMPLE = int((81.74e6 + 7.83e6) / 2)


def load_binding():
    spec = importlib.util.spec_from_file_location("sd3_b200", os.path.join(REPO, "sd3.c_b200", "sd3_b200.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules["sd3_b200"] = mod
    spec.loader.exec_module(mod)
    return mod


def measured_peaks():
    path = os.path.join(REPO, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"],
                    bf16_tflops_sustained=d["bf16_tflops_sustained"], source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.QUERY,
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0, t1):
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
        for ts, line in self.lines:
            if ts < t0 or ts > t1 + 0.1:
                continue
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def device_params(torch, O, device, seed):
    """SD3.5-medium parameters N(0, 0.02), biases 0, generated on the device."""
    c = O.SD35_MEDIUM
    shapes = O.model_param_shapes(c["num_layers"], c["dual_layers"], c["in_dim"], c["E"],
                                  c["pooled_dim"], c["captions_dim"], c["patch"], c["attn_heads"],
                                  c["mlp_expand"])
    gen = torch.Generator(device=device).manual_seed(seed)
    p = {}
    for name, shp in shapes.items():
        if len(shp) >= 2:
            p[name] = (torch.randn(shp, generator=gen, device=device) * 0.02).to(torch.bfloat16)
        elif "rmsnorm" in name:
            p[name] = torch.ones(shp, device=device, dtype=torch.bfloat16)
        else:
            p[name] = torch.zeros(shp, device=device, dtype=torch.bfloat16)
    return p


def time_events(torch, fn, iters, warm=3):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def kernel_breakdown(torch, s, peaks):
    """Times the hot kernels alone at the workload's shapes (CUDA events on the
    launching stream, inputs larger than L2) and relates them to the peaks."""
    dev = "cuda"
    out = []
    tf_peak = peaks["bf16_tflops"]

    def gemm_case(name, M, N, K, count, kind="plain"):
        x = torch.randn(M, K, device=dev).bfloat16()
        w = (torch.randn(N, K, device=dev) * 0.02).bfloat16()
        bias = torch.zeros(N, device=dev)
        if kind == "gate":
            gate = torch.randn(B, N, device=dev)
            resid = torch.zeros(M, N, device=dev)
            fn = lambda: s.check(s.lib().sd3_linear_gate_residual(
                s.ptr(x), s.ptr(w), s.ptr(bias), s.ptr(gate), N, M // B, s.ptr(resid), M, N, K, s.stream_ptr()))
        elif kind == "qkv":
            wq = torch.ones(64, device=dev)
            qkv = torch.empty(B, M // B, N, device=dev, dtype=torch.bfloat16)
            fn = lambda: s.qkv_project(x, w, bias, wq, wq, 1e-6, qkv, B, M // B, M // B, 0, K)
        else:
            o = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
            act = 1 if kind == "gelu" else 0
            fn = lambda: s.check(s.lib().sd3_linear(s.ptr(x), s.ptr(w), s.ptr(bias), s.ptr(o), 1, M, N, K, act, s.stream_ptr()))
        ms = time_events(torch, fn, 10)
        fl = 2.0 * M * N * K
        out.append(dict(kernel=name, launches_per_step=count, ms=round(ms, 4),
                        achieved=round(fl / ms / 1e9, 1), unit="TFLOP/s", bound="tensor",
                        frac=round(fl / ms / 1e9 / tf_peak, 4)))

    Mx = B * TX
    gemm_case("gemm_tcgen05 qkv x (QK-RMSNorm epilogue)", Mx, 3 * E, E, 37, "qkv")
    gemm_case("gemm_tcgen05 out-proj x (gate+residual)", Mx, E, E, 37, "gate")
    gemm_case("gemm_tcgen05 mlp1 x (GELU-tanh)", Mx, FH, E, 24, "gelu")
    gemm_case("gemm_tcgen05 mlp2 x (gate+residual)", Mx, E, FH, 24, "gate")

    def attn_case(name, Tn, Tc, count, bounded=True):
        qkv = normed_qkv(torch, B, Tn, dev, prescale=bounded)
        oc = torch.empty(B, max(Tc, 1), E, device=dev, dtype=torch.bfloat16)
        ox = torch.empty(B, Tn - Tc, E, device=dev, dtype=torch.bfloat16)
        # the step's launches: q and k are RMS-normed by the QKV epilogue (weights 1 in this random-init
        # model), q pre-scaled; the engine passes scale 0 and the bound that follows from the norm weights
        bound, scale = (QK_SCORE_BOUND * QK_PRESCALE, 0.0) if bounded else (0.0, 0.125)
        fn = lambda: s.check(s.lib().sd3_attention_bounded(s.ptr(qkv), B, Tn, NH, Tc, s.ptr(oc) if Tc else None,
                                                           s.ptr(ox), scale, bound, None, 0, s.stream_ptr()))
        ms = time_events(torch, fn, 5)
        fl = 4.0 * B * NH * Tn * Tn * 64
        d = dict(kernel=name, launches_per_step=count, ms=round(ms, 4), achieved=round(fl / ms / 1e9, 1),
                 unit="TFLOP/s", bound="tensor", frac=round(fl / ms / 1e9 / tf_peak, 4))
        out.append(d)
        return d

    joint = attn_case("attention_tcgen05 joint T=4429 (bounded scores, q pre-scaled: as in the step)", T, TC, 24)
    attn_case("attention_tcgen05 image-only T=4096 (bounded scores, q pre-scaled: as in the step)", TX, 0, 13)
    attn_case("attention_tcgen05 joint T=4429, online softmax (no bound given)", T, TC, 0, bounded=False)

    x = torch.randn(Mx, E, device=dev)
    mod = torch.randn(B, 9 * E, device=dev)
    o1 = torch.empty(Mx, E, device=dev, dtype=torch.bfloat16)
    fn = lambda: s.check(s.lib().sd3_layernorm_modulate(s.ptr(x), B, TX, E, 1e-6, mod.data_ptr(), mod[:, E:].data_ptr(),
                                                        s.ptr(o1), None, None, None, 9 * E, 1, s.stream_ptr()))
    ms = time_events(torch, fn, 10)
    by = Mx * E * 6.0
    out.append(dict(kernel="ln_modulate x (fp32 in, bf16 out)", launches_per_step=61, ms=round(ms, 4),
                    achieved=round(by / ms / 1e6, 1), unit="GB/s", bound="hbm",
                    frac=round(by / ms / 1e6 / peaks["hbm_gbs"], 4)))
    # every AdaLN vector of the step: one GEMM with M = batch over the concatenated weights
    N = 502272
    y = torch.randn(B, E, device=dev).bfloat16()
    w = (torch.randn(N, E, device=dev) * 0.02).bfloat16()
    bb = torch.zeros(N, device=dev)
    oo = torch.empty(B, N, device=dev)
    fn = lambda: s.check(s.lib().sd3_linear(s.ptr(y), s.ptr(w), s.ptr(bb), s.ptr(oo), 0, B, N, E, 0, s.stream_ptr()))
    ms = time_events(torch, fn, 10)
    by = N * E * 2.0
    out.append(dict(kernel="gemm_tcgen05 AdaLN, M = batch (all blocks)", launches_per_step=1, ms=round(ms, 4),
                    achieved=round(by / ms / 1e6, 1), unit="GB/s", bound="hbm",
                    frac=round(by / ms / 1e6 / peaks["hbm_gbs"], 4)))
    return out, joint


def profile_step(torch, s):
    """One full denoiser step of the benchmark workload between
    cudaProfilerStart/Stop, after one warm-up step (use a profiler's
    "profile from start off" mode to capture just that step's launch list)."""
    from oracle import mmdit_oracle as O
    dev = torch.device("cuda", 0)
    params = device_params(torch, O, dev, seed=2)
    model = s.Model(24, range(13), 2048, 4096, 16, E, NH, 4, 2, 384, 128, True, s.PRECISION_BF16)
    model.load(params)
    gen = torch.Generator(device=dev).manual_seed(2)
    latent = torch.randn(B, 16, HW, HW, generator=gen, device=dev).bfloat16()
    captions = torch.randn(B, TC, 4096, generator=gen, device=dev).bfloat16()
    pooled = torch.randn(B, 2048, generator=gen, device=dev).bfloat16()
    tsteps = torch.rand(B, generator=gen, device=dev) * 1000
    out = torch.empty_like(latent)
    model.forward(pooled, captions, latent, tsteps, out)
    torch.cuda.synchronize()
    torch.cuda.profiler.start()
    s.lib().sd3_launch_count(1)
    model.forward(pooled, captions, latent, tsteps, out)
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    s.assert_healthy()
    print(json.dumps({"profile_case": "step", "launches": int(s.lib().sd3_launch_count(0))}))


def profile_case(name, reps=3):
    """Runs ONE hot kernel a few times at a reduced size (inputs above L2, well
    under 2 GB) so that a profiler capture of it ends quickly.  Cases:
    gemm_plain, gemm_qkv, gemm_gate, gemm_gelu, attn_joint, attn_self, ln_mod, skinny."""
    import torch
    s = load_binding()
    dev = "cuda"
    torch.manual_seed(0)
    if name == "step":
        return profile_step(torch, s)
    Bp = 2
    M = Bp * TX
    if name.startswith("gemm"):
        N, K = {"gemm_plain": (3 * E, E), "gemm_qkv": (3 * E, E), "gemm_gate": (E, FH), "gemm_gelu": (FH, E)}[name]
        x = torch.randn(M, K, device=dev).bfloat16()
        w = (torch.randn(N, K, device=dev) * 0.02).bfloat16()
        bias = torch.zeros(N, device=dev)
        if name == "gemm_gate":
            gate = torch.randn(Bp, N, device=dev)
            resid = torch.zeros(M, N, device=dev)
            fn = lambda: s.check(s.lib().sd3_linear_gate_residual(
                s.ptr(x), s.ptr(w), s.ptr(bias), s.ptr(gate), N, TX, s.ptr(resid), M, N, K, s.stream_ptr()))
        elif name == "gemm_qkv":
            wq = torch.ones(64, device=dev)
            qkv = torch.empty(Bp, TX, N, device=dev, dtype=torch.bfloat16)
            fn = lambda: s.qkv_project(x, w, bias, wq, wq, 1e-6, qkv, Bp, TX, TX, 0, K)
        else:
            o = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
            act = 1 if name == "gemm_gelu" else 0
            fn = lambda: s.check(s.lib().sd3_linear(s.ptr(x), s.ptr(w), s.ptr(bias), s.ptr(o), 1, M, N, K, act, s.stream_ptr()))
    elif name in ("attn_joint", "attn_self"):
        Tn, Tc = (T, TC) if name == "attn_joint" else (TX, 0)
        qkv = normed_qkv(torch, Bp, Tn, dev)
        oc = torch.empty(Bp, max(Tc, 1), E, device=dev, dtype=torch.bfloat16)
        ox = torch.empty(Bp, Tn - Tc, E, device=dev, dtype=torch.bfloat16)
        fn = lambda: s.check(s.lib().sd3_attention_bounded(s.ptr(qkv), Bp, Tn, NH, Tc, s.ptr(oc) if Tc else None,
                                                           s.ptr(ox), 0.0, QK_SCORE_BOUND * QK_PRESCALE, None, 0,
                                                           s.stream_ptr()))
    elif name == "ln_mod":
        Bl = 8
        x = torch.randn(Bl * TX, E, device=dev)
        mod = torch.randn(Bl, 9 * E, device=dev)
        o1 = torch.empty(Bl * TX, E, device=dev, dtype=torch.bfloat16)
        fn = lambda: s.check(s.lib().sd3_layernorm_modulate(s.ptr(x), Bl, TX, E, 1e-6, mod.data_ptr(), mod[:, E:].data_ptr(),
                                                            s.ptr(o1), None, None, None, 9 * E, 1, s.stream_ptr()))
    elif name == "skinny":
        N = 499200
        y = torch.randn(B, E, device=dev)
        w = (torch.randn(N, E, device=dev) * 0.02).bfloat16()
        bb = torch.zeros(N, device=dev)
        oo = torch.empty(B, N, device=dev)
        fn = lambda: s.check(s.lib().sd3_skinny_linear(s.ptr(y), E, s.ptr(w), 1, s.ptr(bb), None, 0, s.ptr(oo), N, B, N, E, 0, s.stream_ptr()))
    else:
        raise SystemExit("unknown profile case " + name)
    ms = time_events(torch, fn, reps, warm=1)
    s.assert_healthy()
    print(json.dumps({"profile_case": name, "ms": ms}))


def make_config(world):
    """The `config` object of the JSON line; the same for both arms."""
    return {"workload": WORKLOAD, "per_gpu_batch": B / world, "global_batch": B,
            "parallelism": "batch split over %d GPU(s), full weight replica each, no collective" % world,
            "l2": "inputs and activations exceed L2 (126 MB) many times per step"}


def reference_root():
    """Directory of a checkout of the reference, or None: SD3_REFERENCE_ROOT, else a
    directory "reference" next to this repository."""
    root = os.environ.get("SD3_REFERENCE_ROOT") or os.path.join(os.path.dirname(REPO), "reference")
    return root if os.path.exists(os.path.join(root, "module_tests", "modules.py")) else None


class CpuDenoiser:
    """The reference's CPU implementation of the path in bf16 on the host cores:
    its own MMDiT module when a checkout is present (kind "reference"), else
    the oracle's restatement of it (kind "port").  Random N(0, 0.02) weights."""

    def __init__(self, torch, threads):
        self.torch = torch
        torch.set_num_threads(threads)
        self.kind = "port"
        root = reference_root()
        if root is not None:
            try:
                spec = importlib.util.spec_from_file_location("sd3_reference_modules",
                                                              os.path.join(root, "module_tests", "modules.py"))
                ref = importlib.util.module_from_spec(spec)
                spec.loader.exec_module(ref)
                # the reference's sinusoidal embedding returns float32, which its bf16 timestep MLP
                # rejects: hand it on in the dtype of the MLP's weights
                emb = ref.get_sinusoidal_embedding
                ref.get_sinusoidal_embedding = lambda t, emb_dim: emb(t, emb_dim).to(torch.bfloat16)
                gen = torch.Generator().manual_seed(2)
                model = ref.MMDiT(24, list(range(13)), 16, E, 2048, 4096, 2, NH, 4, 384, 128, True)
                with torch.no_grad():
                    for name, prm in model.named_parameters():
                        if prm.dim() >= 2:
                            prm.normal_(0, 0.02, generator=gen)
                        elif "rmsnorm" in name:
                            prm.fill_(1.0)
                        else:
                            prm.zero_()
                self.model = model.to(torch.bfloat16).eval()
                self.kind = "reference"
            except Exception as exc:  # fall back to the port, say why
                sys.stderr.write("reference modules not usable (%s): timing the oracle port\n" % exc)
        if self.kind == "port":
            from oracle import mmdit_oracle as O
            self.O = O
            c = O.SD35_MEDIUM
            shapes = O.model_param_shapes(c["num_layers"], c["dual_layers"], c["in_dim"], c["E"], c["pooled_dim"],
                                          c["captions_dim"], c["patch"], c["attn_heads"], c["mlp_expand"])
            gen = torch.Generator().manual_seed(2)
            self.params = {}
            for name, shp in shapes.items():
                if len(shp) >= 2:
                    self.params[name] = torch.empty(shp, dtype=torch.bfloat16).normal_(0, 0.02, generator=gen)
                elif "rmsnorm" in name:
                    self.params[name] = torch.ones(shp, dtype=torch.bfloat16)
                else:
                    self.params[name] = torch.zeros(shp, dtype=torch.bfloat16)

    def forward_seconds(self, batch):
        """One denoiser forward of `batch` samples at 1024^2; returns seconds."""
        torch = self.torch
        gen = torch.Generator().manual_seed(2)
        latent = torch.randn(batch, 16, HW, HW, generator=gen).bfloat16()
        captions = torch.randn(batch, TC, 4096, generator=gen).bfloat16()
        pooled = torch.randn(batch, 2048, generator=gen).bfloat16()
        t = torch.rand(batch, generator=gen) * 1000
        with torch.no_grad():
            t0 = time.time()
            if self.kind == "reference":
                self.model(latent, captions, pooled, t)
            else:
                self.O.dit_forward(pooled, captions, latent, t, self.params, 24, range(13), 24, 2, 384, 128, True)
            return time.time() - t0


def run_reference(args):
    """Reference arm (rank 0 only): the CPU path on all host threads.  One real batch-8
    forward is timed once; each of the K timed steps is ONE of the eight samples of a
    step (`ms_per_step` is what such a step took)."""
    import torch
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    cpu = CpuDenoiser(torch, threads)
    for _ in range(max(1, min(args.warmup, 2))):
        cpu.forward_seconds(1)
    full = cpu.forward_seconds(B)
    steps = max(1, min(args.steps, 20))
    secs = [cpu.forward_seconds(1) for _ in range(steps)]
    per_sample = sum(secs) / len(secs)
    value = 1.0 / full
    sample = ("one real batch-8 forward timed once (%.1f s, `value`); each of the %d timed steps is one of the "
              "8 samples of a step (B=1, mean %.2f s, i.e. %.4f steps/s if scaled by 8)"
              % (full, steps, per_sample, 1.0 / (per_sample * B)))
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": max(1, min(args.warmup, 2)), "ms_per_step": per_sample * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "config": make_config(max(1, args.gpus)), "device": "host CPU, %d threads" % threads,
        "full_batch_forward_s": full, "sampled_value": 1.0 / (per_sample * B),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": cpu.kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# |q . k| <= 64 max|wq| max|wk| after the per-head RMSNorm; the benchmark model's norm weights are 1
QK_SCORE_BOUND = 1.01 * 64.0


QK_PRESCALE = 0.125 * 1.4426950408889634  # softmax scale * log2(e), folded into q by the engine


def normed_qkv(torch, batch, tokens, dev, prescale=True):
    """Packed (batch, tokens, 3E) bf16 attention input as the engine's QKV epilogue leaves it: q
    and k RMS-normed per head (weights 1), q multiplied by softmax_scale * log2(e), v random."""
    raw = torch.randn(batch, tokens, 3, NH, 64, device=dev)
    raw[:, :, :2] *= torch.rsqrt(raw[:, :, :2].pow(2).mean(-1, keepdim=True) + 1e-6)
    if prescale:
        raw[:, :, 0] *= QK_PRESCALE
    return raw.reshape(batch, tokens, 3 * E).bfloat16()


def library_attention_rows(torch, peaks):
    """Library attention kernels at the benchmark's shapes, as CONTEXT rows of the kernel
    table (not part of the product, nothing here is called on the denoiser's path)."""
    import torch.nn.functional as F
    rows = []
    try:
        from torch.nn.attention import sdpa_kernel, SDPBackend
    except Exception:
        return rows
    for Tn in (T, TX):
        q, k, v = [torch.randn(B, NH, Tn, 64, device="cuda", dtype=torch.bfloat16) for _ in range(3)]
        fl = 4.0 * B * NH * Tn * Tn * 64
        cands = [("torch SDPA, cuDNN backend", lambda: F.scaled_dot_product_attention(q, k, v), SDPBackend.CUDNN_ATTENTION)]
        try:
            from flash_attn import flash_attn_func
            q2, k2, v2 = [t.transpose(1, 2).contiguous() for t in (q, k, v)]
            cands.append(("flash_attn (mma.sync)", lambda: flash_attn_func(q2, k2, v2), None))
        except Exception:
            pass
        for name, fn, backend in cands:
            try:
                if backend is not None:
                    with sdpa_kernel(backend):
                        ms = time_events(torch, fn, 5)
                else:
                    ms = time_events(torch, fn, 5)
                rows.append(dict(kernel="[library, context only] %s T=%d" % (name, Tn), launches_per_step=0,
                                 ms=round(ms, 4), achieved=round(fl / ms / 1e9, 1), unit="TFLOP/s", bound="tensor",
                                 frac=round(fl / ms / 1e9 / peaks["bf16_tflops"], 4)))
            except Exception as exc:
                rows.append(dict(kernel="[library, context only] %s T=%d" % (name, Tn), error=str(exc)[:100]))
    return rows


def time_region(torch, dist, fn, steps, dev):
    """`steps` calls of fn between CUDA events, max over ranks; returns total ms."""
    torch.cuda.synchronize()
    if dist:
        dist.barrier()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if dist:
        tms = torch.tensor([ms], device=dev)
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
        ms = tms.item()
        dist.barrier()
    return ms


def long_sequence_case(torch, s, dist, params, model, dev, rank, world):
    """One 2048x2048 image (16384 image + 333 context tokens): the fused one-GPU forward on
    rank 0 and, with more than one rank, the token-sharded forward (all-to-all around every
    attention), checked against the one-GPU result in the same run."""
    gen = torch.Generator(device=dev).manual_seed(4)
    lat = torch.randn(1, 16, 256, 256, generator=gen, device=dev).bfloat16()
    cap = torch.randn(1, TC, 4096, generator=gen, device=dev).bfloat16()
    pool = torch.randn(1, 2048, generator=gen, device=dev).bfloat16()
    tt = torch.rand(1, generator=gen, device=dev) * 1000
    if world > 1:  # every rank must hold the same inputs
        for tns in (lat, cap, pool, tt):
            dist.broadcast(tns, 0)
    out1 = torch.empty_like(lat)
    fwd1 = lambda: model.forward(pool, cap, lat, tt, out1)
    for _ in range(2):
        fwd1()
    ms1 = time_region(torch, dist, fwd1, 3, dev) / 3
    res = {"workload": "one 2048^2 image, 16384 image + 333 context tokens, batch 1, bf16",
           "n_gpus": world, "ms_1gpu": round(ms1, 3)}
    if world == 1:
        res["ms"] = res["ms_1gpu"]
        return res
    spec = importlib.util.spec_from_file_location("sd3_ulysses", os.path.join(REPO, "sd3.c_b200", "ulysses.py"))
    uly = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(uly)
    cfg = dict(num_layers=24, dual_attention_layers=list(range(13)), pooled_dim=2048, captions_dim=4096,
               in_channels=16, emb_dim=E, attn_heads=NH, mlp_expand=4, patch_size=2, pos_embed_max_size=384,
               base_height=128)
    pm = uly.PackedModel(s, params, cfg)
    comm = uly.DistComm()
    fwd = lambda: uly.dit_forward_sharded(pm, pool, cap, lat, tt, comm)
    outp = fwd()
    fwd()
    msp = time_region(torch, dist, fwd, 3, dev) / 3
    rel = ((outp.float() - out1.float()).norm() / out1.float().norm()).item()
    Tl = 16384 // world
    # per attention and rank: q|k|v of the local image rows out (all but the own head group),
    # and the attention output of the local heads back, bf16
    a2a = 37 * (Tl * 3 * E * 2 + Tl * E * 2) * (world - 1) // world
    res.update({"ms": round(msp, 3), "speedup_vs_1gpu": round(ms1 / msp, 3), "rel_l2_vs_1gpu": rel,
                "a2a_bytes_per_step_per_gpu": a2a})
    del pm
    return res


def sampling_loop_case(torch, s, dist, params, model, dev, rank, world, with_fp8):
    """The 28-step Euler flow-matching loop with classifier-free guidance (conditional and
    unconditional branches stacked: effective batch 2 x images), 16 images at 1024^2 split
    over the ranks, guidance 4.5, shift-3 schedule.  The schedule is this repository's own
    (the reference has no sampler): what is measured is the denoiser under its caller."""
    lo, hi = s.shard_range(16, world, rank)
    n = hi - lo
    gen = torch.Generator(device=dev).manual_seed(40 + rank)
    lat = torch.randn(n, 16, HW, HW, generator=gen, device=dev).bfloat16()
    cc = torch.randn(n, TC, 4096, generator=gen, device=dev).bfloat16()
    cp = torch.randn(n, 2048, generator=gen, device=dev).bfloat16()
    uc = torch.zeros_like(cc)
    up = torch.zeros_like(cp)
    out = []
    models = [("bf16", model)]
    if with_fp8:
        m8 = s.Model(24, range(13), 2048, 4096, 16, E, NH, 4, 2, 384, 128, True, s.PRECISION_FP8)
        m8.load(params)
        models.append(("fp8_e4m3 block GEMMs", m8))
    for name, mdl in models:
        mdl.reserve(2 * n, TC, HW, HW)
        s.sample(mdl, lat, cc, cp, uc, up, steps=1)  # warm-up (workspace, kernel attributes)
        ms = time_region(torch, dist, lambda: s.sample(mdl, lat, cc, cp, uc, up, steps=28, guidance=4.5, shift=3.0), 1, dev)
        out.append({"precision": name, "s_per_loop": round(ms / 1e3, 3), "images_per_s": round(16.0 / (ms / 1e3), 3),
                    "images": 16, "images_per_gpu": n, "steps": 28, "effective_batch_per_gpu": 2 * n})
    if with_fp8:
        models[1][1].close()
    s.assert_healthy()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--precision", choices=["bf16", "fp8"], default="bf16",
                    help="fp8: block GEMMs on e4m3 operands (an extra mode; the headline metric is bf16)")
    ap.add_argument("--no-breakdown", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the c4 / c5 / extension legs")
    ap.add_argument("--no-graph", action="store_true",
                    help="device-resident loop: launch the kernels one by one instead of replaying a CUDA graph")
    ap.add_argument("--profile-case", default=None,
                    help="run one hot kernel a few times at a reduced size (for profiler captures)")
    args = ap.parse_args()
    if args.profile_case:
        return profile_case(args.profile_case)
    if args.impl == "reference":
        return run_reference(args)

    import torch
    from oracle import mmdit_oracle as O  # parameter shapes only
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the denoiser has no CPU path")
    s = load_binding()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local)
    peaks = measured_peaks()
    warm = max(args.warmup, 3)

    params = device_params(torch, O, dev, seed=2)
    model = s.Model(24, range(13), 2048, 4096, 16, E, NH, 4, 2, 384, 128, True,
                    s.PRECISION_FP8 if args.precision == "fp8" else s.PRECISION_BF16)
    model.load(params)
    model.reserve(B, TC, HW, HW)
    # the whole batch of 8 (same on every rank); rank r owns samples [lo, hi)
    gen = torch.Generator(device=dev).manual_seed(2)
    latent = torch.randn(B, 16, HW, HW, generator=gen, device=dev).bfloat16()
    captions = torch.randn(B, TC, 4096, generator=gen, device=dev).bfloat16()
    pooled = torch.randn(B, 2048, generator=gen, device=dev).bfloat16()
    tsteps = torch.rand(B, generator=gen, device=dev) * 1000
    out = torch.empty_like(latent)
    lo, hi = s.shard_range(B, world, rank)
    nb = hi - lo
    sl = slice(lo, hi)
    my = [t[sl].contiguous() for t in (pooled, captions, latent, tsteps)]
    my_out = torch.empty_like(my[2])

    # The device-resident loop calls the denoiser on fixed device buffers, so it replays the
    # forward as one CUDA graph (Model.forward_graphed; --no-graph launches the kernels one by
    # one): the same kernels in the same order, without the host's launch calls between them.
    fwd = model.forward if args.no_graph else model.forward_graphed

    def step():  # this rank's share of one batch-8 step
        if nb > 0:
            fwd(my[0], my[1], my[2], my[3], my_out)

    def step_whole():  # a whole batch of 8 on this rank
        fwd(pooled, captions, latent, tsteps, out)

    # ---- device-resident timing: the batch of 8 split over the ranks --------------
    for _ in range(warm):
        step()
    torch.cuda.synchronize()
    s.assert_healthy()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    s.lib().sd3_launch_count(1)
    t_wall0 = time.time()
    ms = time_region(torch, dist, step, args.steps, dev)
    t_wall1 = time.time()
    launches = s.lib().sd3_launch_count(0)
    if not args.no_graph and nb > 0:  # replayed launches do not pass the library's counter
        launches = args.steps * model.graph_launches(my[0], my[1], my[2], my[3], my_out)
    clocks = sampler.stop(t_wall0, t_wall1) if rank == 0 else None
    s.assert_healthy()
    ms_per_step = ms / args.steps
    value = 1000.0 / ms_per_step
    # every rank a whole batch of 8 (identical to the above at one GPU)
    if world > 1:
        for _ in range(2):
            step_whole()
        ms_w = time_region(torch, dist, step_whole, args.steps, dev) / args.steps
    else:
        ms_w = ms_per_step
    weak_value = world * 1000.0 / ms_w

    # ---- end to end: host buffers in, host buffer out, through the serving call --
    h_in = [t.cpu().pin_memory() for t in my]
    h_out = torch.empty(my_out.shape, dtype=my_out.dtype).pin_memory()
    e2e_value, h2d, d2h = None, 0, 0
    pipe = None
    if nb > 0:
        # HostPipeline.submit uploads the batch on a copy stream, runs the denoiser, downloads
        # the result; with two device input sets the copies of neighbouring steps overlap the
        # compute.  All of it is inside the timed region (the last download is waited for).
        pipe = s.HostPipeline(model, nb, TC, 16, HW, HW, 2048, 4096, torch.bfloat16, depth=2,
                              use_graph=not args.no_graph)

    def e2e_run():
        if pipe is not None:
            for _ in range(args.steps):
                pipe.submit(h_in[0], h_in[1], h_in[2], h_in[3], h_out)
            pipe.flush()

    if pipe is not None:
        for _ in range(2):
            pipe.submit(h_in[0], h_in[1], h_in[2], h_in[3], h_out)
        pipe.flush()
    ms2 = time_region(torch, dist, e2e_run, 1, dev)
    e2e_value = 1000.0 * args.steps / ms2
    # bytes of the whole batch-8 step over all ranks
    h2d = sum(t.numel() * t.element_size() for t in (latent, captions, pooled, tsteps))
    d2h = out.numel() * out.element_size()
    del pipe

    # ---- end to end through the drop-in torch extension (rank 0, its share) ------
    ext = None
    if not args.no_extras and rank == 0 and nb > 0:
        try:
            if os.path.join(REPO, "sd3.c_b200") not in sys.path:
                sys.path.insert(0, os.path.join(REPO, "sd3.c_b200"))
            import custom_modules
            pdict = {k: v for k, v in params.items()}

            def ext_step():
                o = custom_modules.DiT(h_in[0].to(dev, non_blocking=True), h_in[1].to(dev, non_blocking=True),
                                       h_in[2].to(dev, non_blocking=True), h_in[3].to(dev, non_blocking=True), pdict,
                                       24, set(range(13)), 2048, 4096, 16, E, NH, 4, 2, 384, 128, True)
                h_out.copy_(o, non_blocking=True)

            for _ in range(2):
                ext_step()
            torch.cuda.synchronize()
            n_ext = max(3, args.steps // 2)
            e0 = torch.cuda.Event(enable_timing=True)
            e1 = torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(n_ext):
                ext_step()
            e1.record()
            torch.cuda.synchronize()
            ext = {"call": "custom_modules.DiT on pinned host tensors -> .to(device) -> DiT -> host copy",
                   "ms_per_call": round(e0.elapsed_time(e1) / n_ext, 3), "samples_per_call": nb,
                   "value_rank0_share": round(1000.0 * n_ext / e0.elapsed_time(e1), 4)}
            del pdict
        except Exception as exc:
            ext = {"error": str(exc)[:200]}

    # ---- the other workloads of the reference's scope (extra keys) ---------------
    c5 = c4 = None
    if not args.no_extras and args.precision == "bf16":
        c5 = long_sequence_case(torch, s, dist, params, model, dev, rank, world)
        c4 = sampling_loop_case(torch, s, dist, params, model, dev, rank, world, with_fp8=True)

    if rank != 0:
        if dist:
            dist.destroy_process_group()
        return

    # ---- per-kernel roofline (rank 0, kernels timed alone) -----------------------
    step_tf = STEP_TFLOP / (ms_per_step / 1e3) / world
    kernels, joint = (None, None)
    if not args.no_breakdown:
        model.close()
        del params
        torch.cuda.empty_cache()
        kernels, joint = kernel_breakdown(torch, s, peaks)
        kernels += library_attention_rows(torch, peaks)
    if joint is not None:
        roofline = {"bound": "tensor", "kernel": "attention_tcgen05_kernel (joint, T=4429, B=8, 24 heads)",
                    "achieved": joint["achieved"], "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                    "frac": joint["frac"], "traffic": ATTN_TRAFFIC_BYTES_PER_SAMPLE * B,
                    "traffic_source": "ncu dram__bytes_read+write of the batch-2 capture in profiles/, per sample x batch",
                    "peak_source": peaks["source"] + " burst"}
    else:
        roofline = {"bound": "tensor", "kernel": "whole step", "achieved": round(step_tf, 1),
                    "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s",
                    "frac": round(step_tf / peaks["bf16_tflops_sustained"], 4), "traffic": None,
                    "peak_source": peaks["source"] + " sustained"}

    # ---- CPU baseline (rank 0, N=1 only): bounded sample on the host cores -------
    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        torch.cuda.empty_cache()
        den = CpuDenoiser(torch, threads)
        den.forward_seconds(1)
        secs = den.forward_seconds(1)
        cpu = {"value": 1.0 / (secs * B), "unit": UNIT, "cores": threads, "kind": den.kind,
               "sample": "one forward of 1 of the 8 samples (B=1, 1024^2, bf16) on the host cores after one "
                         "warm-up forward; step time = 8 x %.2f s (the reference arm times a real batch-8 forward)" % secs}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": warm, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16" if args.precision == "bf16" else "fp8_e4m3 block GEMMs, bf16 elsewhere (not the headline precision)",
        "data": "synthetic",
        "config": make_config(world),
        "weak_value": weak_value, "weak_ms_per_step": ms_w,
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "call": "sd3_b200.HostPipeline.submit (pinned host batch -> sd3_dit_forward -> pinned host)"},
        "e2e_extension": ext,
        "gpu_launches": int(launches),
        "launch_mode": "kernel by kernel" if args.no_graph else "one CUDA graph replay per step (value and e2e); e2e_extension kernel by kernel",
        "clocks": clocks,
        "step_tflops_per_gpu": round(step_tf, 1),
        "step_frac_of_sustained_peak": round(step_tf / peaks["bf16_tflops_sustained"], 4),
        "step_frac_of_burst_peak": round(step_tf / peaks["bf16_tflops"], 4),
        "step_frac_of_nominal_2250": round(step_tf / 2250.0, 4),
        "roofline": roofline,
        "cpu_baseline": cpu,
        "c5": c5, "c4": c4,
        "kernels": kernels,
    }
    print(json.dumps(line))
    if dist:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
