#!/usr/bin/env python
"""Benchmark of the gradient + Hessian-vector hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one computeCNNGradient + one cnnHv on one synthetic batch per GPU:
VGG-11-BN, fp64, 512 images of 3x32x32 per GPU (weak scaling: at 8 GPUs this is the
4096-image configuration the metric is quoted on).  Inputs are seeded synthetic data
(N(0,1) images, uniform labels, He-normal weights, N(0,1) direction); the models come from the
library's own builders (fitre_read_vgg11 and friends).

Prints ONE JSON line: images/s over all GPUs (device-resident inputs, CUDA events, max over
ranks), the same metric end to end through the host-buffer C-ABI entry point (`e2e`), the
roofline of the dominant kernel (implicit-GEMM convolution, fp64 tensor path) with its
duration measured by CUDA events inside the timed region, on 1 GPU the CPU baseline, and in
`secondary` the device-timed figures of the path's other configurations at the same GPU count
(LeNet gradient + Hv + 10 Steihaug-CG iterations, AlexNet-BN gradient + Hv at a global batch of
1024, the KFAC step at 256 images per GPU).  With more than one GPU, `multi_gpu_parity` holds
the relative errors of a small sharded problem against the full-batch oracle, and
`e2e_node_shared_results` the end-to-end figure when the ranks of the node share one page-locked
result segment and upload the replicated inputs in chunks (extra information; `e2e` keeps
private buffers and full transfers on every rank).

`--impl reference` times the same step on the host cores: the gradient and the Hessian-vector
product by double backward as PyTorch computes them on the CPU (the operator of the
reference's pytorch/ path), all threads, one full per-GPU batch per step; the C + OpenMP port
of the reference's CUDA host code (oracle/) is timed beside it on a bounded sample and the
faster of the two is the reported value.
"""
import argparse
import ctypes as C
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
PORT_SAMPLE_IMAGES = 256     # oracle port (C + OpenMP): one pass, ~7-15 s on 16 cores
TORCH_SAMPLE_IMAGES = 256    # PyTorch-on-CPU leg of the default run
DMMA_FMA_PER_CLK_SM = 64     # fp64 tensor-pipe issue limit of one SM (FMA per clock)
N_SM = 148


# ---- models (the library's own builders) ----------------------------------------------------
def product_model(kind, n):
    from fitre_b200 import api
    from fitre_b200 import _structs as S
    if kind == "vgg11":      # nn/read_vgg.c:216-299: no bias, batch norm, Swish, max pooling
        return api.readVGG11(n, 32, 32, 10, 3, 0, 1, S.CNN_ACT_SWISH)
    if kind == "alexnet":    # nn/read_alexnet.c:14-243 topology with batch norm
        return api.readAlexNetCNN(n, 32, 32, 10, 0, 1, S.CNN_ACT_SWISH)
    if kind == "lenet":      # nn/read_nn.c:500-725 topology; ReLU + max pooling as the configuration states
        return api.readLenetCNN(3, 32, 32, n, 1, 0, S.CNN_ACT_RELU, S.MAX_POOL)
    raise ValueError(kind)


def bench_config(n, world):
    return {"workload": WORKLOAD, "per_gpu_batch": n, "global_batch": n * world,
            "parallelism": "dp%d" % world, "activation": "swish", "batch_norm": True,
            "l2": "inputs larger than L2 (z/dx/rz are 1.85 GiB each per GPU)"}


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


# ---- CPU legs ---------------------------------------------------------------------------------
def host_threads():
    return os.cpu_count() or 1


def use_all_host_threads():
    """torch.distributed.run exports OMP_NUM_THREADS=1 to its workers; the CPU legs use every
    core, so the variable is set before an OpenMP runtime reads it and the oracle library is
    told explicitly as well."""
    os.environ["OMP_NUM_THREADS"] = str(host_threads())


def checker_model(n):
    """VGG-11-BN description for the CPU legs, built without the CUDA library (test-side net
    description + the oracle's own offset computation; byte-identical to fitre_read_vgg11's)."""
    import nets
    import oracle_lib as O
    m = nets.vgg11(n)
    O.finalize(m)
    return m


def cpu_oracle_rate(sample_images):
    """images/s of one gradient + one Hv of the oracle port on the host cores."""
    use_all_host_threads()
    import oracle_lib as O
    try:
        O.lib().ora_set_num_threads(host_threads())
    except AttributeError:
        pass
    m = checker_model(sample_images)
    x, y, w, v = synth(m, sample_images, 4321)
    t0 = time.perf_counter()
    st = O.gradient(m, x, y, w, 10, sample_images)
    O.hv(m, x, w, 10, sample_images, st, v)
    dt = time.perf_counter() - t0
    return sample_images / dt, dt


def cpu_pytorch_step(case):
    """One gradient + Hessian-vector product as PyTorch runs it on the host cores: fp64 autograd
    gradient and double backward, the operator of the reference's pytorch/ path
    (pytorch/kfac/alexnet_cifar.py:297-324).  Returns the seconds of the step."""
    import torch_ref
    m, x, y, w, v, n = case
    t0 = time.perf_counter()
    torch_ref.loss_grad_hv(m, w, x, y, n, vectors=(v,))
    return time.perf_counter() - t0


def cpu_pytorch_case(n):
    import torch
    torch.set_num_threads(host_threads())
    m = checker_model(n)
    x, y, w, v = synth(m, n, 4321)
    return m, x, y, w, v, n


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    use_all_host_threads()
    world = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
    n = args.per_gpu_batch
    cores = host_threads()
    line = {
        "impl": "reference", "metric": "gradient+Hv images/sec", "unit": "images/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f64",
        "data": "synthetic", "config": bench_config(n, world), "gpu_launches": 0,
    }
    # the C + OpenMP port of the reference's CUDA host code, one bounded pass
    port_rate, port_dt = cpu_oracle_rate(PORT_SAMPLE_IMAGES)
    line["cpu_baseline_port"] = {"value": port_rate, "unit": "images/s", "cores": cores, "kind": "port",
                                 "sample": "%d images, C + OpenMP restatement of the reference's CUDA host "
                                           "code (%.1f s)" % (PORT_SAMPLE_IMAGES, port_dt)}
    value, ms, kind, sample = port_rate, 1e3 * port_dt * n / PORT_SAMPLE_IMAGES, "port", line["cpu_baseline_port"]["sample"]
    try:
        case = cpu_pytorch_case(n)
        first = cpu_pytorch_step(case)
        warm, steps = args.warmup, args.steps
        if first * (warm + steps) > 600.0:
            # this host would need more than ten minutes: one warm-up step and what fits four minutes
            warm, steps = min(warm, 1), max(1, min(steps, int(240.0 / first)))
            line["steps"], line["warmup"] = steps, warm
        times = [first] if warm == 0 else []
        for _ in range(max(warm - 1, 0)):
            cpu_pytorch_step(case)
        while len(times) < steps:
            times.append(cpu_pytorch_step(case))
        t_rate = n * len(times) / sum(times)
        line["cpu_baseline_pytorch"] = {"value": t_rate, "unit": "images/s", "cores": cores,
                                        "sample": "%d steps of one %d-image batch each" % (len(times), n)}
        if t_rate >= port_rate:
            value, ms, kind = t_rate, 1e3 * sum(times) / len(times), "port"
            sample = ("%d-image batches, fp64 autograd gradient + double-backward Hessian-vector product in "
                      "PyTorch on the host cores (the operator of the reference's pytorch/ path, restated "
                      "for current PyTorch); faster than the C + OpenMP port (%.1f images/s)" % (n, port_rate))
    except Exception as e:  # noqa: BLE001 -- a missing or failing torch CPU path leaves the port figure
        line["cpu_baseline_pytorch"] = {"unavailable": str(e)[:200]}
    line.update({"value": value, "ms_per_step": ms,
                 "cpu_baseline": {"value": value, "unit": "images/s", "cores": cores, "kind": kind, "sample": sample},
                 "e2e": {"value": value, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}})
    print(json.dumps(line), flush=True)


# ---- secondary workloads (the path's other configurations) -----------------------------------
SECONDARY_NAMES = {"alexnet": "alexnetbn_32x32_fp64_gradient+hv",
                   "lenet": "lenet_32x32_fp64_gradient+hv+cg10",
                   "kfac": "vgg11bn_32x32_fp64_kfac_step(grad,sampled bwd,A/G factors,factorisations,natural gradient)"}


def time_secondary(ctx, wl, world, rank, steps, warmup, kfac_solver="cholesky", graphs=True, one_call=False):
    """Device-timed steps of one secondary workload at the current rank count.
    alexnet: gradient + Hv, AlexNet-BN, 1024 images over the ranks (strong scaling);
    lenet: gradient, Hv and 10 Steihaug-CG iterations at 256 images per GPU;
    kfac: VGG-11-BN KFAC step, 256 images per GPU (gradient, sampled-label backward, A and G
    factors, 22 damped factorisations, natural gradient; layer-owned factors with ranks)."""
    import torch
    import torch.distributed as dist
    from fitre_b200 import _lib, api
    from fitre_b200 import _structs as S
    L = _lib.load()
    n = {"alexnet": max(1, 1024 // world), "lenet": 256, "kfac": 256}[wl]
    model = product_model({"kfac": "vgg11"}.get(wl, wl), n)
    x, y, w, v = synth(model, n, 2234 + rank)
    _, _, w, v = synth(model, n, 2234)
    f64 = dict(dtype=torch.float64, device="cuda")
    X, Y, W, V = (torch.tensor(a, **f64) for a in (x, y, w, v))
    data = api.make_dataset(W, X, Y, 10)
    ws = api.Workspace(model, 10)
    extra = {}
    if wl == "kfac":
        ctx.set_kfac_solver(1 if kfac_solver == "cholesky" else 0)
        ctx.set_graphs(graphs)
        ctx.set_kfac_distribution(1)  # with ranks: factors stay on a layer's owner rank
        extra["kfac_solver"], extra["cuda_graphs"] = kfac_solver, bool(graphs)
        extra["factor_calls"] = "one call after the sampled-label pass" if one_call else \
            "A side started before the sampled-label pass, G side after it"
        if world > 1:
            extra["kfac_distribution"] = "layer_owned"
        info = api.computeKFACStorageIndices(model)
        kscr = torch.zeros(max(L.fitre_kfac_mem_required(C.byref(model)), ws.dev.numel()), **f64)
        A, G = torch.zeros(info.OmegaZSize, **f64), torch.zeros(info.LambdaGSize, **f64)
        Ai, Gi = torch.zeros(info.OmegaZSize, **f64), torch.zeros(info.LambdaGSize, **f64)
        U, tgt = torch.rand(n, **f64), torch.zeros(n, **f64)
        md = model.maxDeltaSize + 32
        e1b, e2b = torch.zeros(md, **f64), torch.zeros(md, **f64)
        dgrad, ddx = torch.zeros(model.pSize, **f64), torch.zeros(model.zSize, **f64)
        ngrad = torch.zeros(model.pSize, **f64)
        iscr = torch.zeros(max(L.fitre_kfac_factors_and_inverses_mem_required(C.byref(model)),
                               L.fitre_kfac_natural_gradient_mem_required(C.byref(model))), **f64)
        info.regLambda, info.dampGamma = 1e-3, 0.0
    elif wl == "lenet":
        p = torch.zeros(model.pSize, **f64)

    def step():
        api.computeCNNGradient(ctx, model, data, ws.scratch, ws.z, ws.dx, ws.probs, ws.errors,
                               ws.gradient, 0, n, 0.0)
        if wl == "alexnet":
            api.cnnHv(ctx, model, data, ws.z, ws.probs, ws.errors, ws.dx, V, ws.hv, 0, n, ws.dev)
        elif wl == "lenet":
            api.cnnHv(ctx, model, data, ws.z, ws.probs, ws.errors, ws.dx, V, ws.hv, 0, n, ws.dev)
            prm = S.CG_PARAMS()
            # H + 500 I is positive definite for this net, so all ten iterations run
            prm.delta, prm.tolerance, prm.maxIterations, prm.weightDecay = 1e3, 1e-30, 10, 500.0
            api.cgSteihaug(ctx, model, data, ws.z, ws.probs, ws.errors, ws.dx, ws.gradient, p,
                           n, ws.dev, prm)
            extra["cg_iterations"], extra["cg_hv_calls"] = prm.iterations, prm.hvCalls
        elif one_call:
            api.computeDistributionErrors(ctx, ws.probs, U, tgt, e1b, n, 10)
            api.cnnBackward(ctx, model, data, kscr, ws.z, dgrad, ddx, e1b, e2b, 0, n)
            # A/G factors and the 22 damped factorisations (inverses or Cholesky), overlapped
            api.computeFactorsAndInverses(ctx, model, data, ws.z, ddx, n, A, Ai, G, Gi, info, iscr)
            api.computeNaturalGradient(ctx, model, info, Ai, Gi, ws.gradient, ngrad, iscr)
        else:
            # A factors and their factorisation chains start on the library's own streams and run
            # underneath the sampled-label backward pass; the G side joins them afterwards
            api.computeOmegaZBegin(ctx, model, data, ws.z, n, A, Ai, info, iscr)
            api.computeDistributionErrors(ctx, ws.probs, U, tgt, e1b, n, 10)
            api.cnnBackward(ctx, model, data, kscr, ws.z, dgrad, ddx, e1b, e2b, 0, n)
            api.computeLambdaDeltaFinish(ctx, model, ddx, n, G, Gi, info, iscr)
            api.computeNaturalGradient(ctx, model, info, Ai, Gi, ws.gradient, ngrad, iscr)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    try:
        for _ in range(warmup):
            step()
        barrier()
        l0 = ctx.launches
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        launches = ctx.launches - l0
    finally:
        if wl == "kfac":
            ctx.set_kfac_solver(0)
            ctx.set_kfac_distribution(0)
            ctx.set_graphs(True)
    if world > 1:
        t = torch.tensor([ms], **f64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    images = n * world
    return {"workload": SECONDARY_NAMES[wl], "value": images * steps / (ms * 1e-3), "unit": "images/s",
            "ms_per_step": ms / steps, "steps": steps, "warmup": warmup, "per_gpu_batch": n,
            "global_batch": images, "scaling": {"alexnet": "strong", "lenet": "weak", "kfac": "weak"}[wl],
            "gpu_launches": launches, **extra}


def multi_gpu_parity(ctx, world, rank):
    """A small sharded problem against the full-batch oracle: vgg_small with batch norm, 8 images per
    rank.  Every rank evaluates its shard through the library (sync batch norm, all-reduced
    gradient / Hv / A factors); rank 0 evaluates the whole batch with the CPU oracle and reports the
    relative differences.  Outside every timed region."""
    import torch
    from fitre_b200 import _lib, api, layout
    from fitre_b200 import _structs as S

    def small_vgg(batch):  # conv3 + BN + Swish three times, max pooling after the first and third
        sw, mp = S.CNN_ACT_SWISH, (S.MAX_POOL, 2, 2, 0)
        convs = [dict(cin=3, cout=8, h=8, w=8, k=3, pad=1, bn=True, act=sw, pool=mp),
                 dict(cin=8, cout=8, h=4, w=4, k=3, pad=1, bn=True, act=sw, pool=None),
                 dict(cin=8, cout=16, h=4, w=4, k=3, pad=1, bn=True, act=sw, pool=mp)]
        return api.finalize(S.describe_model(convs, [(16 * 2 * 2, 10, S.CNN_ACT_NONE)], batch, False))

    per = 8
    n_glob = per * world
    full = small_vgg(n_glob)
    x, y, w, v = synth(full, n_glob, 2024)
    c0 = full.convLayer[0]
    xs = layout.shard_batch(x, n_glob, c0.inChannels, c0.height, c0.width, rank, world)
    ys = np.ascontiguousarray(y[rank * per:(rank + 1) * per])
    model = small_vgg(per)
    f64 = dict(dtype=torch.float64, device="cuda")
    X, Y, W, V = (torch.tensor(a, **f64) for a in (xs, ys, w, v))
    data = api.make_dataset(W, X, Y, 10)
    ws = api.Workspace(model, 10)
    loss = api.computeCNNGradient(ctx, model, data, ws.scratch, ws.z, ws.dx, ws.probs, ws.errors,
                                  ws.gradient, 0, per, 0.0)
    api.cnnHv(ctx, model, data, ws.z, ws.probs, ws.errors, ws.dx, V, ws.hv, 0, per, ws.dev)
    info = api.computeKFACStorageIndices(model)
    A = torch.zeros(info.OmegaZSize, **f64)
    kscr = torch.zeros(_lib.load().fitre_kfac_mem_required(C.byref(model)), **f64)
    api.computeOmegaZ(ctx, model, data, ws.z, per, A, info, kscr)
    g, hv, A = ws.gradient.cpu().numpy(), ws.hv.cpu().numpy(), A.cpu().numpy()
    if rank != 0:
        return None
    import oracle_lib as O
    st = O.gradient(full, x, y, w, 10, n_glob)
    hv_o = O.hv(full, x, w, 10, n_glob, st, v)
    info_o = S.KFAC_INFO()
    O.lib().ora_kfac_storage_indices(C.byref(full), C.byref(info_o))
    A_o = np.zeros(info_o.OmegaZSize)
    env = O.make_env()
    O.lib().ora_kfac_omega_z(C.byref(env), C.byref(full), x, st.z, n_glob, A_o, C.byref(info_o))
    rel = lambda a, b: float(np.linalg.norm(a - b) / np.linalg.norm(b))
    k1 = full.convLayer[1].inChannels * 9
    a0 = info_o.OmegaZOffsets[1]
    return {"case": "vgg_small with batch norm, %d images per rank, %d ranks, against the full-batch CPU oracle" % (per, world),
            "loss_rel": abs(loss - st.loss) / abs(st.loss), "gradient_rel": rel(g, st.gradient),
            "hv_rel": rel(hv, hv_o), "kfac_A_layer1_rel": rel(A[a0:a0 + k1 * k1], A_o[a0:a0 + k1 * k1]),
            "tolerance": 1e-10}


def bind_to_gpu_numa_node(gpu_index):
    """With several ranks on one box, run this process on the CPU cores next to its GPU (NVML's
    topology query) before the pinned host buffers are allocated, so that host-to-device and
    device-to-host copies stay on the local socket.  What `numactl --cpunodebind` would do for a
    user; reads NVML, changes only this process's CPU affinity.  Returns the core count or None."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(gpu_index)
        words = (host_threads() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(h, words)
        cpus = [64 * i + b for i, wd in enumerate(mask) for b in range(64) if (int(wd) >> b) & 1]
        allowed = os.sched_getaffinity(0)
        cpus = [c for c in cpus if c in allowed]
        if cpus:
            os.sched_setaffinity(0, cpus)
            return len(cpus)
    except Exception:  # noqa: BLE001 -- best effort: no NVML, no affinity support
        pass
    return None


def time_shared_results(ctx, model, api, hx, hy, hw, hv_in, hg, hh, n, world, rank, args, barrier, e0, e1,
                        h2d, d2h):
    """End to end like `e2e`, with gradient and Hv delivered once per node into a segment all ranks
    share; checks afterwards that the shared vectors are the private-buffer results bit for bit."""
    import torch
    import torch.distributed as dist
    P = model.pSize
    shm = "/dev/shm/fitre_bench_%s" % os.environ.get("MASTER_PORT", "0")
    # rank 0 creates the segment if the node's shared-memory file system has room for it (touching a
    # tmpfs mapping beyond its limit is a bus error, not an exception) and tells the others
    ok = torch.zeros(1, dtype=torch.float64, device="cuda")
    if rank == 0:
        try:
            st = os.statvfs("/dev/shm")
            if st.f_bavail * st.f_frsize > 2 * P * 8 + (64 << 20):
                np.memmap(shm, dtype=np.float64, mode="w+", shape=(2 * P,)).flush()
                ok[0] = 1.0
        except OSError:
            pass
    dist.broadcast(ok, 0)
    if float(ok.item()) != 1.0:
        return {"skipped": "no room for a %d MB segment in /dev/shm" % (2 * P * 8 >> 20)}
    buf = np.memmap(shm, dtype=np.float64, mode="r+", shape=(2 * P,))
    rt = torch.cuda.cudart()
    rt.cudaHostRegister(buf.ctypes.data, buf.nbytes, 0)
    ctx.set_host_results_shared(1)
    ctx.set_host_inputs_replicated(1)  # weights and direction are the same on every rank
    try:
        def host_step():
            return api.gradientHvHost(ctx, model, hx, hy, hw, hv_in, n, 10, 0.0, buf[:P], buf[P:])
        for _ in range(max(1, min(args.warmup, 3))):
            host_step()
        barrier()
        e0.record()
        for _ in range(args.steps):
            host_step()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        same = bool(np.array_equal(np.asarray(buf[:P]), hg.numpy()) and np.array_equal(np.asarray(buf[P:]), hh.numpy()))
    finally:
        ctx.set_host_results_shared(0)
        ctx.set_host_inputs_replicated(0)
        rt.cudaHostUnregister(buf.ctypes.data)
        dist.barrier()
        del buf
        if rank == 0:
            os.unlink(shm)
    return {"value": world * n * args.steps / (ms * 1e-3), "unit": "images/s", "ms_per_step": ms / args.steps,
            "h2d_bytes_per_step_per_rank": h2d - (world - 1) * d2h // world,
            "d2h_bytes_per_step_per_rank": d2h // world,
            "results_equal_private_buffers": same,
            "note": "weights, direction, gradient and Hv cross PCIe once per node: every rank uploads a 1/%d "
                    "chunk of the replicated inputs (all-gathered over NVLink) and copies its share of the "
                    "results into a page-locked segment that all ranks read" % world}


# ---- the benchmark ----------------------------------------------------------------------------
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
    numa_cores = bind_to_gpu_numa_node(local) if world > 1 else None
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if args.gpus != world and rank == 0:
        sys.stderr.write("bench.py: --gpus %d but WORLD_SIZE %d; using WORLD_SIZE\n" % (args.gpus, world))

    n = args.per_gpu_batch
    model = product_model("vgg11", n)
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

    # ---- the same with ONE result buffer per node: the ranks' processes map and page-lock the same
    # shared-memory segment, each copies its 1/world share of gradient and Hv, all find the whole
    # vectors (fitre_set_host_results_shared).  Extra information; `e2e` above stays the figure with
    # private buffers on every rank.
    e2e_shared = None
    if world > 1:
        try:
            e2e_shared = time_shared_results(ctx, model, api, hx, hy, hw, hv_in, hg, hh, n, world, rank, args,
                                             barrier, e0, e1, h2d, d2h)
        except Exception as e:  # noqa: BLE001 -- extra information must not take the headline down
            e2e_shared = {"error": str(e)[:300]}

    # ---- the path's other configurations at this GPU count, and the sharded-parity check
    secondary, parity = {}, None
    if not args.no_secondary and args.precision == "fp64":
        del X, Y, data
        torch.cuda.empty_cache()
        for wl, st_, wu_ in (("lenet", 5, 2), ("alexnet", 3, 2), ("kfac", 3, 2)):
            try:
                secondary[wl] = time_secondary(ctx, wl, world, rank, st_, wu_)
            except Exception as e:  # noqa: BLE001 -- a secondary figure must not take the headline down
                secondary[wl] = {"workload": SECONDARY_NAMES[wl], "error": str(e)[:300]}
            torch.cuda.empty_cache()
        if world > 1:
            try:
                parity = multi_gpu_parity(ctx, world, rank)
            except Exception as e:  # noqa: BLE001
                parity = {"error": str(e)[:300]}

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
    sm_mhz = (clocks or {}).get("sm_mhz") or 1965.0
    issue_limit = 2.0 * DMMA_FMA_PER_CLK_SM * N_SM * sm_mhz * 1e6 / 1e12
    cfg = bench_config(n, world)   # the reference arm prints the same object
    line = {
        "metric": "gradient+Hv images/sec", "value": value, "unit": "images/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f64" if args.precision == "fp64" else args.precision, "data": "synthetic",
        "config": cfg,
        "roofline": {"bound": "tensor",
                     "kernel": "conv_tma_kernel (TMA-fed implicit-GEMM fprop/dgrad, fp64 DMMA; gather kernel for layer 0)"
                     if args.precision == "fp64" else
                     "conv_tf32_kernel (tcgen05 %s fprop/dgrad; fp64 kernels for layer 0 and the weight "
                     "gradients; shown against the fp64 DGEMM peak for comparison with the default mode)"
                     % args.precision,
                     "achieved": achieved, "peak": dgemm_tflops, "unit": "TFLOP/s",
                     "frac": (achieved / dgemm_tflops) if achieved else None,
                     "peak_source": "cuBLAS DGEMM 8192^3 measured in this run (MEASURED_PEAKS.json has no fp64 figure)",
                     # the same against the instruction-issue limit of the fp64 tensor pipe, which no
                     # measured probe can flatter: 64 FMA per clock per SM x 148 SMs x the sampled SM clock
                     "issue_limit": issue_limit,
                     "frac_of_issue_limit": (achieved / issue_limit) if achieved else None,
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
        "algorithmic_mflop_per_image": {"gradient": gpi / 1e6, "hv": hpi / 1e6},
    }
    if e2e_shared is not None:
        line["e2e_node_shared_results"] = e2e_shared
    if world > 1:
        line["multi_gpu"] = {
            "host_binding": ("process bound to the %d cores next to its GPU" % numa_cores) if numa_cores else "none",
            "small_allreduce": "own kernel over peer memory" if ctx.peer_reduce_enabled else "nccl",
            "slice_allreduce": "per layer on a second communicator and stream"}
    if secondary:
        line["secondary"] = secondary
    if parity is not None:
        line["multi_gpu_parity"] = parity
    if world == 1 and not args.skip_cpu:
        r, dt = cpu_oracle_rate(PORT_SAMPLE_IMAGES)
        port = {"value": r, "unit": "images/s", "cores": host_threads(), "kind": "port",
                "sample": "%d images of the same VGG-11-BN fp64 gradient+Hv step, C + OpenMP port of the "
                          "reference's CUDA host code (%.1f s of CPU work)" % (PORT_SAMPLE_IMAGES, dt)}
        line["cpu_baseline"] = port
        try:  # the same step in PyTorch on the host cores; the faster leg is the reported baseline
            case = cpu_pytorch_case(TORCH_SAMPLE_IMAGES)
            dtt = cpu_pytorch_step(case)
            rt = TORCH_SAMPLE_IMAGES / dtt
            torch_leg = {"value": rt, "unit": "images/s", "cores": host_threads(), "kind": "port",
                         "sample": "%d images, fp64 autograd gradient + double-backward Hv in PyTorch on the "
                                   "host cores, the operator of the reference's pytorch/ path (%.1f s)"
                                   % (TORCH_SAMPLE_IMAGES, dtt)}
            line["cpu_baseline_pytorch"] = torch_leg
            if rt > r:
                line["cpu_baseline"], line["cpu_baseline_port"] = torch_leg, port
        except Exception as e:  # noqa: BLE001 -- a missing or failing torch CPU path must not fail the bench
            line["cpu_baseline_pytorch"] = {"unavailable": str(e)[:200]}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_extra(args):
    """One secondary workload by itself (`--workload alexnet|lenet|kfac`): one JSON line, device
    timing only."""
    import torch
    import torch.distributed as dist
    from fitre_b200 import api
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ctx = api.Context(local)
    if world > 1:
        ctx.comm_init_from_torch()
    r = time_secondary(ctx, args.workload, world, rank, args.steps, args.warmup, args.kfac_solver,
                       not args.no_graphs, args.kfac_one_call)
    if world > 1:
        dist.destroy_process_group()
    if rank == 0:
        cfg = {k: r[k] for k in r if k not in ("value", "unit", "ms_per_step", "steps", "warmup", "gpu_launches",
                                                "scaling")}
        print(json.dumps({
            "metric": "images/sec", "value": r["value"], "unit": "images/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["ms_per_step"],
            "higher_is_better": True, "scaling": r["scaling"], "dtype": "f64", "data": "synthetic",
            "config": cfg, "gpu_launches": r["gpu_launches"]}), flush=True)


def run_fitre(args):
    """The FITRE outer loop (trust-region KFAC) on VGG-11-BN, 256 images per GPU: time per
    minibatch of the whole loop body -- device minibatch assembly with augmentation, gradient,
    sampled-label backward, A/G factors, damped inverses, natural gradient, two quadratic models
    (two Hessian-vector products), weight update, re-evaluation -- as the library's own loop runs it."""
    import torch
    import torch.distributed as dist
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
    model = product_model("vgg11", n)
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
                         "for one of the path's other configurations by itself")
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
    ap.add_argument("--kfac-one-call", action="store_true",
                    help="kfac workload: factors and factorisations in one call after the sampled-label "
                         "backward pass instead of starting the A side before it")
    ap.add_argument("--skip-cpu", action="store_true",
                    help="leave the CPU baseline leg out (profiling runs)")
    ap.add_argument("--no-secondary", action="store_true",
                    help="leave the secondary workloads and the sharded-parity check out (profiling runs)")
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
