#!/usr/bin/env python
"""Benchmark of the gradient + Hessian-vector hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one computeCNNGradient + one cnnHv on one synthetic batch per GPU:
VGG-11-BN, fp64, 512 images of 3x32x32 per GPU (weak scaling: at 8 GPUs this is the
4096-image configuration the metric is quoted on).  Inputs are seeded synthetic data
(N(0,1) images, uniform labels, He-normal weights, N(0,1) direction).

Prints ONE JSON line: images/s over all GPUs (device-resident inputs, CUDA events, max over
ranks), the same metric end to end through the host-buffer C-ABI entry point (`e2e`), the
roofline of the dominant kernel (implicit-GEMM convolution, fp64 tensor path) with its
duration measured by CUDA events inside the timed region, and on 1 GPU the CPU baseline
(the oracle port on the host cores, bounded sample).

`--impl reference` times the reference path's CPU restatement (oracle/) with all host
threads on a bounded sample of the same workload and prints the same line shape.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)

import numpy as np  # noqa: E402

PER_GPU_BATCH = 512
WORKLOAD = "vgg11bn_32x32_fp64_gradient+hv"
# algorithmic flops per image (2*M*K*Cout products only): gradient 913.1 MF + Hv 1819.1 MF
TORCH_SAMPLE_IMAGES = 256    # PyTorch-on-CPU leg beside it
CPU_SAMPLE_IMAGES = 256      # cpu_baseline leg of the default run: one pass, ~15 s on 16 cores
REF_SAMPLE_IMAGES = 64       # --impl reference: per timed step


def build_model(n):
    import nets
    from fitre_b200 import api
    m = nets.vgg11(n)
    api.finalize(m)
    return m


def synth(model, n, seed):
    from fitre_b200 import layout
    rng = np.random.default_rng(seed)
    c0 = model.convLayer[0]
    x = layout.batch_to_ref(rng.standard_normal((n, c0.inChannels, c0.height, c0.width)))
    y = rng.integers(1, 11, n).astype(np.float64)
    w = layout.he_normal_params(model, rng)
    v = rng.standard_normal(model.pSize)
    return x, y, w, v


def conv_flops_per_image(model):
    """Algorithmic conv/FC flops of one gradient and one Hv per image."""
    g = h = 0.0
    for l in range(model.cLayers):
        c = model.convLayer[l]
        mkc = 2.0 * c.outHeight * c.outWidth * c.inChannels * c.kSize ** 2 * c.outChannels
        g += (2 if l == 0 else 3) * mkc
        h += (2 if l == 0 else 6) * mkc
    for l in range(model.lLayers):
        f = model.fcLayer[l]
        g += 3 * 2.0 * f.in_ * f.out
        h += 6 * 2.0 * f.in_ * f.out
    return g, h


class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.p = None
        try:
            self.p = subprocess.Popen(["nvidia-smi", "-i", str(gpu_index), "--query-gpu=" + self.QUERY,
                                       "--format=csv,noheader,nounits", "-lms", "100"],
                                      stdout=self.f, stderr=subprocess.DEVNULL)
        except OSError:
            self.p = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.p is None:
            return out
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except Exception:
            self.p.kill()
        self.f.flush()
        self.f.seek(0)
        sm, mx, reasons = [], [], set()
        for line in self.f.read().splitlines():
            parts = [t.strip() for t in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                  "sw_power_cap"), parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        try:
            os.unlink(self.f.name)
        except OSError:
            pass
        if sm:
            # samples under load: the upper half of the clock samples
            sm_sorted = sorted(sm)
            out["sm_mhz"] = statistics.median(sm_sorted[len(sm_sorted) // 2:])
            out["sm_max_mhz"] = max(mx)
            out["samples"] = len(sm)
        out["reasons"] = sorted(reasons)
        return out


def cpu_oracle_rate(sample_images, threads=None):
    """images/s of one gradient + one Hv of the oracle port on the host cores."""
    import oracle_lib as O
    import nets
    if threads:
        os.environ["OMP_NUM_THREADS"] = str(threads)
    m = nets.vgg11(sample_images)
    O.finalize(m)
    x, y, w, v = synth(m, sample_images, 4321)
    t0 = time.perf_counter()
    st = O.gradient(m, x, y, w, 10, sample_images)
    O.hv(m, x, w, 10, sample_images, st, v)
    dt = time.perf_counter() - t0
    return sample_images / dt, dt


def cpu_pytorch_rate(sample_images):
    """images/s of the same step as PyTorch runs it on the host cores: fp64 autograd gradient and
    Hessian-vector product by double backward, the operator of the reference's pytorch/ path
    (pytorch/kfac/alexnet_cifar.py:297-324), all threads."""
    import torch
    import nets
    import oracle_lib as O
    import torch_ref
    torch.set_num_threads(os.cpu_count() or 1)
    m = nets.vgg11(sample_images)
    O.finalize(m)
    x, y, w, v = synth(m, sample_images, 4321)
    t0 = time.perf_counter()
    torch_ref.loss_grad_hv(m, w, x, y, sample_images, vectors=(v,))
    dt = time.perf_counter() - t0
    return sample_images / dt, dt


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    rates = []
    for i in range(args.warmup + args.steps):
        r, dt = cpu_oracle_rate(REF_SAMPLE_IMAGES)
        if i >= args.warmup:
            rates.append((r, dt))
    value = REF_SAMPLE_IMAGES * len(rates) / sum(dt for _, dt in rates)
    line = {
        "impl": "reference", "metric": "gradient+Hv images/sec", "value": value, "unit": "images/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * sum(dt for _, dt in rates) / len(rates),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f64",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, "per_gpu_batch": PER_GPU_BATCH,
                   "note": "CPU restatement of the reference path (oracle/, C + OpenMP); each step "
                           "is a %d-image sample of the workload" % REF_SAMPLE_IMAGES},
        "cpu_baseline": {"value": value, "unit": "images/s", "cores": cores, "kind": "port",
                         "sample": "%d images of the VGG-11-BN fp64 gradient+Hv step" % REF_SAMPLE_IMAGES},
        "e2e": {"value": value, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    try:  # the same step as PyTorch runs it on the host cores, for comparison with the port
        rt, dtt = cpu_pytorch_rate(TORCH_SAMPLE_IMAGES)
        line["cpu_baseline_pytorch"] = {"value": rt, "unit": "images/s", "cores": cores,
                                        "sample": "%d images (%.1f s)" % (TORCH_SAMPLE_IMAGES, dtt)}
    except Exception as e:  # noqa: BLE001
        line["cpu_baseline_pytorch"] = {"unavailable": str(e)[:200]}
    print(json.dumps(line), flush=True)


def run_ours(args):
    import torch
    import torch.distributed as dist
    from fitre_b200 import api

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device (the product path has no CPU fallback)")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if args.gpus != world and rank == 0:
        sys.stderr.write("bench.py: --gpus %d but WORLD_SIZE %d; using WORLD_SIZE\n" % (args.gpus, world))

    n = args.per_gpu_batch
    model = build_model(n)
    ctx = api.Context(local)
    if world > 1:
        ctx.comm_init_from_torch()
    if args.precision != "fp64":
        ctx.set_precision({"tf32": 1, "tf32x3": 2, "fp64i8": 3}[args.precision])
    x, y, w, v = synth(model, n, 3234 + rank)   # each rank holds its own shard of the batch
    _, _, w, v = synth(model, n, 3234)          # parameters and direction are replicated
    f64 = dict(dtype=torch.float64, device="cuda")
    X, Y = torch.tensor(x, **f64), torch.tensor(y, **f64)
    W, V = torch.tensor(w, **f64), torch.tensor(v, **f64)
    data = api.make_dataset(W, X, Y, 10)
    ws = api.Workspace(model, 10)

    def step():
        api.computeCNNGradient(ctx, model, data, ws.scratch, ws.z, ws.dx, ws.probs, ws.errors,
                               ws.gradient, 0, n, 0.0)
        api.cnnHv(ctx, model, data, ws.z, ws.probs, ws.errors, ws.dx, V, ws.hv, 0, n, ws.dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local) if rank == 0 else None  # nvidia-smi needs ~1 s to start
    for _ in range(args.warmup):
        step()
    barrier()
    launches0 = ctx.launches
    ctx.profile_enable(True)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    ctx.profile_enable(False)
    launches = ctx.launches - launches0
    k_ms, k_flops, k_n = ctx.profile_read(0)
    w_ms, w_flops, w_n = ctx.profile_read(1)
    clocks = sampler.stop() if sampler else None
    if world > 1:
        t = torch.tensor([ms], **f64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    value = world * n * args.steps / (ms * 1e-3)

    # ---- end to end through the host-buffer C-ABI entry point (pinned host memory)
    hx = torch.tensor(x).pin_memory()
    hy = torch.tensor(y).pin_memory()
    hw = torch.tensor(w).pin_memory()
    hv_in = torch.tensor(v).pin_memory()
    hg = torch.zeros(model.pSize, dtype=torch.float64).pin_memory()
    hh = torch.zeros(model.pSize, dtype=torch.float64).pin_memory()
    del ws
    torch.cuda.empty_cache()

    def host_step():
        return api.gradientHvHost(ctx, model, hx, hy, hw, hv_in, n, 10, 0.0, hg, hh)

    for _ in range(max(1, min(args.warmup, 3))):
        host_step()
    barrier()
    t0 = time.perf_counter()
    e0.record()
    for _ in range(args.steps):
        host_step()
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([e2e_ms], **f64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_value = world * n * args.steps / (e2e_ms * 1e-3)
    h2d = 8 * (x.size + y.size + w.size + v.size)
    d2h = 8 * 2 * model.pSize

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- fp64 tensor peak: cuBLAS DGEMM 8192^3 measured in this run (burst, best of 5)
    a = torch.randn(8192, 8192, **f64)
    b = torch.randn(8192, 8192, **f64)
    torch.matmul(a, b)
    best = 1e30
    for _ in range(5):
        e0.record()
        torch.matmul(a, b)
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1))
    dgemm_tflops = 2.0 * 8192 ** 3 / (best * 1e-3) / 1e12
    del a, b

    achieved = (k_flops / (k_ms * 1e-3)) / 1e12 if k_ms > 0 else None
    gpi, hpi = conv_flops_per_image(model)
    line = {
        "metric": "gradient+Hv images/sec", "value": value, "unit": "images/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f64" if args.precision == "fp64" else args.precision, "data": "synthetic",
        "config": {"workload": WORKLOAD, "per_gpu_batch": n, "global_batch": n * world,
                   "parallelism": "dp%d" % world, "activation": "swish", "batch_norm": True,
                   "l2": "inputs larger than L2 (z/dx/rz are 1.85 GiB each per GPU)",
                   "algorithmic_mflop_per_image": {"gradient": gpi / 1e6, "hv": hpi / 1e6}},
        "roofline": {"bound": "tensor",
                     "kernel": "conv_tma_kernel (TMA-fed implicit-GEMM fprop/dgrad, fp64 DMMA; gather kernel for layer 0)"
                     if args.precision == "fp64" else
                     "conv_tf32_kernel (tcgen05 %s fprop/dgrad; fp64 kernels for layer 0 and the weight "
                     "gradients; shown against the fp64 DGEMM peak for comparison with the default mode)"
                     % args.precision,
                     "achieved": achieved, "peak": dgemm_tflops, "unit": "TFLOP/s",
                     "frac": (achieved / dgemm_tflops) if achieved else None,
                     "peak_source": "cuBLAS DGEMM 8192^3 measured in this run (MEASURED_PEAKS.json has no fp64 figure)",
                     "launches": k_n, "avg_launch_ms": k_ms / max(k_n, 1),
                     "share_of_step": k_ms / ms,
                     # dram__bytes_read+write of the layer-3 forward launch, ncu capture at 256
                     # images scaled by 2 (profiles/conv_tma_kernel_vgg11bn_n256.md); its
                     # algorithmic bytes (input + weights + output) are 138.9 MB
                     "traffic": 116.8e6 if n == PER_GPU_BATCH else None,
                     "traffic_launch": "layer 3 forward (M 32768, K 2304, Cout 256)",
                     "wgrad_kernel": {"achieved": (w_flops / (w_ms * 1e-3)) / 1e12 if w_ms > 0 else None,
                                      "launches": w_n, "share_of_step": w_ms / ms}},
        "e2e": {"value": e2e_value, "unit": "images/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms / args.steps},
        "gpu_launches": launches,
        "clocks": clocks,
        "per_gpu_algorithmic_tflops": (gpi + hpi) * n * args.steps / (ms * 1e-3) / 1e12,
    }
    if world == 1 and not args.skip_cpu:
        r, dt = cpu_oracle_rate(CPU_SAMPLE_IMAGES)
        line["cpu_baseline"] = {"value": r, "unit": "images/s", "cores": os.cpu_count() or 1,
                                "kind": "port",
                                "sample": "%d images of the same VGG-11-BN fp64 gradient+Hv step "
                                          "(%.1f s of CPU work)" % (CPU_SAMPLE_IMAGES, dt)}
        try:  # the same step in PyTorch on the host cores, reported beside the port
            rt, dtt = cpu_pytorch_rate(TORCH_SAMPLE_IMAGES)
            line["cpu_baseline_pytorch"] = {
                "value": rt, "unit": "images/s", "cores": os.cpu_count() or 1,
                "sample": "%d images, fp64 autograd gradient + double-backward Hv (%.1f s)"
                          % (TORCH_SAMPLE_IMAGES, dtt)}
        except Exception as e:  # noqa: BLE001 -- a missing or failing torch CPU path must not fail the bench
            line["cpu_baseline_pytorch"] = {"unavailable": str(e)[:200]}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_extra(args):
    """Secondary workloads (the other configurations of the path): one JSON line each, device
    timing only.  alexnet: gradient+Hv, AlexNet-BN, 1024 images over the ranks; lenet: gradient,
    Hv and 10 Steihaug-CG iterations at 256 images; kfac: VGG-11-BN KFAC factor step (gradient,
    sampled-label backward, A and G factors), 256 images per GPU."""
    import ctypes as C
    import torch
    import torch.distributed as dist
    import nets
    from fitre_b200 import _lib, api
    from fitre_b200 import _structs as S
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ctx = api.Context(local)
    if world > 1:
        ctx.comm_init_from_torch()
    wl = args.workload
    n = {"alexnet": 1024 // world, "lenet": 256, "kfac": 256}[wl]
    model = {"alexnet": nets.alexnet, "lenet": nets.lenet, "kfac": nets.vgg11}[wl](n)
    api.finalize(model)
    x, y, w, v = synth(model, n, 2234 + rank)
    _, _, w, v = synth(model, n, 2234)
    f64 = dict(dtype=torch.float64, device="cuda")
    X, Y, W, V = (torch.tensor(a, **f64) for a in (x, y, w, v))
    data = api.make_dataset(W, X, Y, 10)
    ws = api.Workspace(model, 10)
    extra = {}
    if wl == "kfac":
        ctx.set_kfac_solver(1 if args.kfac_solver == "cholesky" else 0)
        ctx.set_graphs(not args.no_graphs)
        ctx.set_kfac_distribution(1)  # with ranks: factors stay on a layer's owner rank
        extra["kfac_solver"], extra["cuda_graphs"] = args.kfac_solver, not args.no_graphs
        if world > 1:
            extra["kfac_distribution"] = "layer_owned"
        info = api.computeKFACStorageIndices(model)
        need = _lib.load().fitre_kfac_mem_required(C.byref(model))
        kscr = torch.zeros(max(need, ws.dev.numel()), **f64)
        A = torch.zeros(info.OmegaZSize, **f64)
        G = torch.zeros(info.LambdaGSize, **f64)
        U = torch.rand(n, **f64)
        tgt = torch.zeros(n, **f64)
        md = model.maxDeltaSize + 32
        e1b, e2b = torch.zeros(md, **f64), torch.zeros(md, **f64)
        dgrad, ddx = torch.zeros(model.pSize, **f64), torch.zeros(model.zSize, **f64)
        Ai, Gi = torch.zeros(info.OmegaZSize, **f64), torch.zeros(info.LambdaGSize, **f64)
        ngrad = torch.zeros(model.pSize, **f64)
        L = _lib.load()
        iscr = torch.zeros(max(L.fitre_kfac_factors_and_inverses_mem_required(C.byref(model)),
                               L.fitre_kfac_natural_gradient_mem_required(C.byref(model))), **f64)
        info.regLambda, info.dampGamma = 1e-3, 0.0
        blocks = []
        for l in range(model.cLayers + model.lLayers):
            if l < model.cLayers:
                c = model.convLayer[l]
                kb, co = c.inChannels * c.kSize ** 2 + model.bias, c.outChannels
            else:
                f = model.fcLayer[l - model.cLayers]
                kb, co = f.in_ + model.bias, f.out
            blocks.append((kb, info.OmegaZOffsets[l], A, Ai))
            blocks.append((co, info.LambdaGOffsets[l], G, Gi))

    def step():
        api.computeCNNGradient(ctx, model, data, ws.scratch, ws.z, ws.dx, ws.probs, ws.errors,
                               ws.gradient, 0, n, 0.0)
        if wl == "alexnet":
            api.cnnHv(ctx, model, data, ws.z, ws.probs, ws.errors, ws.dx, V, ws.hv, 0, n, ws.dev)
        elif wl == "lenet":
            api.cnnHv(ctx, model, data, ws.z, ws.probs, ws.errors, ws.dx, V, ws.hv, 0, n, ws.dev)
            prm = S.CG_PARAMS()
            prm.delta, prm.tolerance, prm.maxIterations, prm.weightDecay = 1e3, 1e-30, 10, 1.0
            api.cgSteihaug(ctx, model, data, ws.z, ws.probs, ws.errors, ws.dx, ws.gradient, ws.hv,
                           n, ws.dev, prm)
            extra["cg_iterations"], extra["cg_hv_calls"] = prm.iterations, prm.hvCalls
        else:
            api.computeDistributionErrors(ctx, ws.probs, U, tgt, e1b, n, 10)
            api.cnnBackward(ctx, model, data, kscr, ws.z, dgrad, ddx, e1b, e2b, 0, n)
            # A/G factors and the 22 damped factorisations (inverses or Cholesky), overlapped
            api.computeFactorsAndInverses(ctx, model, data, ws.z, ddx, n, A, Ai, G, Gi, info, iscr)
            api.computeNaturalGradient(ctx, model, info, Ai, Gi, ws.gradient, ngrad, iscr)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    l0 = ctx.launches
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], **f64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        dist.destroy_process_group()
    if rank == 0:
        names = {"alexnet": "alexnetbn_32x32_fp64_gradient+hv",
                 "lenet": "lenet_32x32_fp64_gradient+hv+cg10",
                 "kfac": "vgg11bn_32x32_fp64_kfac_step(grad,sampled bwd,A/G factors,inverses,natural gradient)"}
        print(json.dumps({
            "metric": "images/sec", "value": world * n * args.steps / (ms * 1e-3), "unit": "images/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "strong" if wl == "alexnet" else "weak", "dtype": "f64", "data": "synthetic",
            "config": dict({"workload": names[wl], "per_gpu_batch": n}, **extra),
            "gpu_launches": ctx.launches - l0}), flush=True)


def run_fitre(args):
    """The FITRE outer loop (trust-region KFAC) on VGG-11-BN, 256 images per GPU: time per
    minibatch of the whole loop body -- device minibatch assembly with augmentation, gradient,
    sampled-label backward, A/G factors, damped inverses, natural gradient, two quadratic models
    (two Hessian-vector products), weight update, re-evaluation -- as the library's own loop runs it."""
    import ctypes as C
    import numpy as np
    import torch
    import torch.distributed as dist
    import nets
    from fitre_b200 import _lib, api
    from fitre_b200 import _structs as S
    from fitre_b200 import layout
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ctx = api.Context(local)
    if world > 1:
        ctx.comm_init_from_torch()
    ctx.set_kfac_solver(1 if args.kfac_solver == "cholesky" else 0)
    ctx.set_graphs(not args.no_graphs)
    n = 256
    model = nets.vgg11(n)
    api.finalize(model)
    mbs = args.warmup + args.steps
    n_train = (mbs + 1) * n * world        # the loop stops before the batch that reaches the end
    rng = np.random.default_rng(99)        # same synthetic CIFAR-shaped set on every rank
    f64 = dict(dtype=torch.float64, device="cuda")
    trainX = torch.tensor(rng.integers(0, 256, n_train * 3072).astype(np.float64), **f64)
    trainY = torch.tensor(rng.integers(1, 11, n_train).astype(np.float64), **f64)
    W = torch.tensor(layout.he_normal_params(model, rng), **f64)
    data = api.make_full_dataset(W, trainX, trainY, None, None, 10, 3072, n)
    need = _lib.load().fitre_trust_region_kfac_mem_required(C.byref(model), C.byref(data), None)
    scr = api.make_scratch(torch.zeros(need, **f64))

    def run(count):
        info = S.KFAC_INFO()
        info.regLambda, info.dampGamma, info.momentum, info.checkGrad, info.inverseFreq = 1e-3, 1e-2, 0.9, 1, 1
        tr = S.TRUST_REGION_PARAMS()
        tr.delta, tr.minDelta, tr.maxDelta, tr.maxIters = 0.05, 1e-6, 10.0, 1
        l0 = ctx.launches
        steps, epochs = api.subsampledTrustRegionKFAC(ctx, model, data, info, tr, scr, seed=3, enableDA=1,
                                                      maxMiniBatches=count, stepsCap=count)
        return steps, epochs[0], ctx.launches - l0

    # generalisation sweep after the epoch is part of the call; keep it small by timing the sweep apart
    run(args.warmup)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    steps, ep, launches = run(args.steps)
    secs = torch.tensor([ep.seconds], **f64)
    if world > 1:
        dist.all_reduce(secs, op=dist.ReduceOp.MAX)
    ms = float(secs.item()) * 1e3 / max(ep.miniBatches, 1)
    if rank == 0:
        print(json.dumps({
            "metric": "images/sec", "value": world * n / (ms * 1e-3), "unit": "images/s", "n_gpus": world,
            "steps": ep.miniBatches, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "dtype": "f64", "data": "synthetic",
            "config": {"workload": "vgg11bn_32x32_fp64_fitre_loop_minibatch", "per_gpu_batch": n,
                       "kfac_solver": args.kfac_solver,
                       "timing": "host clock around the minibatch sweep inside the library call, max over ranks"},
            "first_loss": steps[0].trainLikelihood, "last_loss": steps[-1].newTrainLikelihood,
            "kfac_steps": sum(s.usedKfac for s in steps), "reverted": sum(s.reverted for s in steps),
            "gpu_launches": launches}), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="vgg11", choices=["vgg11", "alexnet", "lenet", "kfac", "fitre"],
                    help="vgg11 = the benchmark (default); the others print a device-timed line "
                         "for the path's other configurations")
    ap.add_argument("--per-gpu-batch", type=int, default=PER_GPU_BATCH,
                    help="images per GPU (default 512, the benchmark shape; smaller values are "
                         "for profiler captures only)")
    ap.add_argument("--precision", default="fp64", choices=["fp64", "tf32", "tf32x3", "fp64i8"],
                    help="fp64 = the reference's arithmetic (default, the benchmark); tf32 / tf32x3 = "
                         "the opt-in tcgen05 modes (one TF32 product / error-compensated three), "
                         "reported under their own dtype and never as the headline")
    ap.add_argument("--kfac-solver", default="cholesky", choices=["inverse", "cholesky"],
                    help="kfac / fitre workloads: explicit damped inverses of the A blocks (the "
                         "reference's form) or Cholesky factors applied by triangular solves")
    ap.add_argument("--no-graphs", action="store_true",
                    help="kfac / fitre workloads: launch the factorisation and natural-gradient "
                         "sequences kernel by kernel instead of replaying their CUDA graphs")
    ap.add_argument("--skip-cpu", action="store_true",
                    help="leave the CPU baseline leg out (profiling runs)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "fitre":
        run_fitre(args)
    elif args.workload != "vgg11":
        run_extra(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
