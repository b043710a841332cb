"""Worker used by the multi-rank tests: each rank evaluates its shard of one batch and the
per-rank results are combined by sum all-reduce (gloo + the CPU oracle, or NCCL + the CUDA
library).  Run as a child process: python multirank_worker.py <backend> <rank> <world> <port> <out.npz>
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
for p in (ROOT, HERE):
    if p not in sys.path:
        sys.path.insert(0, p)

N_GLOBAL = 8


def make_case(builder="vgg_small"):
    import nets
    import oracle_lib as O
    from fitre_b200 import layout
    rng = np.random.default_rng(2024)
    model_full = getattr(nets, builder)(N_GLOBAL)
    O.finalize(model_full)
    c0 = model_full.convLayer[0]
    ncls = model_full.fcLayer[model_full.lLayers - 1].out
    x = layout.batch_to_ref(rng.standard_normal((N_GLOBAL, c0.inChannels, c0.height, c0.width)))
    y = rng.integers(1, ncls + 1, N_GLOBAL).astype(np.float64)
    w = layout.he_normal_params(model_full, rng)
    v = rng.standard_normal(model_full.pSize)
    return model_full, x, y, w, v, ncls


def loop_case(per_rank_batch):
    """Inputs of the outer-loop test: a small image set and a vgg_small laid out for one rank."""
    from test_training_oracle import loop_params, small_problem
    rng = np.random.default_rng(77)
    model, trainX, trainY, testX, testY, w = small_problem(rng, n_train=60, n_test=21,
                                                          batch=per_rank_batch)
    info, tr = loop_params()
    return model, trainX, trainY, testX, testY, w, info, tr


def pack_loop(steps, epochs, w):
    f = lambda rows, names: np.array([[getattr(r, n) for n in names] for r in rows], dtype=np.float64)
    return dict(steps=f(steps, ["trainLikelihood", "newTrainLikelihood", "newTrainAccuracy", "modelKfac",
                                "modelGradient", "rho", "delta", "usedKfac", "reverted"]),
                epochs=f(epochs, ["testLikelihood", "testAccuracy", "trainLikelihood", "trainAccuracy",
                                  "miniBatches"]), w=w)


def run_loop(backend, rank, world, out):
    """Each rank runs the FITRE loop on its slices of every global minibatch."""
    import torch
    import torch.distributed as dist
    import oracle_lib as O
    model, trainX, trainY, testX, testY, w, info, tr = loop_case(8 // world)
    if backend == "gloo":
        dist.init_process_group("gloo", rank=rank, world_size=world)

        def allreduce(buf, n, user):
            dist.all_reduce(torch.from_numpy(np.ctypeslib.as_array(buf, shape=(n,))))

        env = O.make_env(world=world, allreduce=allreduce, rank=rank)
        steps, epochs = O.trust_region_kfac(model, trainX, trainY, testX, testY, w, 10, info, tr, seed=5,
                                            steps_cap=64, env=env)
        np.savez(out, **pack_loop(steps, epochs, w))
    else:
        import ctypes as C
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        import gpu_util as G
        from fitre_b200 import api, _lib
        ctx = api.Context(rank)
        ctx.comm_init_from_torch()
        c0 = model.convLayer[0]
        W = G.dev(w)
        data = api.make_full_dataset(W, G.dev(trainX), G.dev(trainY), G.dev(testX), G.dev(testY), 10,
                                     c0.inChannels * c0.height * c0.width, model.batchSize)
        need = _lib.load().fitre_trust_region_kfac_mem_required(C.byref(model), C.byref(data), None)
        scr = api.make_scratch(torch.zeros(need, dtype=torch.float64, device="cuda"))
        steps, epochs = api.subsampledTrustRegionKFAC(ctx, model, data, info, tr, scr, seed=5, stepsCap=64)
        np.savez(out, **pack_loop(steps, epochs, W.cpu().numpy()))
        torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()


def main():
    backend, rank, world, port, out = sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), sys.argv[4], sys.argv[5]
    builder = sys.argv[6] if len(sys.argv) > 6 else "vgg_small"
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=port, RANK=str(rank), WORLD_SIZE=str(world))
    if builder == "loop":
        return run_loop(backend, rank, world, out)
    import torch
    import torch.distributed as dist
    import nets
    import oracle_lib as O
    from fitre_b200 import layout
    model_full, x, y, w, v, ncls = make_case(builder)
    c0 = model_full.convLayer[0]
    per = N_GLOBAL // world
    xs = layout.shard_batch(x, N_GLOBAL, c0.inChannels, c0.height, c0.width, rank, world)
    ys = np.ascontiguousarray(y[rank * per:(rank + 1) * per])
    model = getattr(nets, builder)(per)
    O.finalize(model)
    if backend == "gloo":
        dist.init_process_group("gloo", rank=rank, world_size=world)

        def allreduce(buf, n, user):
            a = np.ctypeslib.as_array(buf, shape=(n,))
            t = torch.from_numpy(a)
            dist.all_reduce(t)

        env = O.make_env(ref_softmax=1, world=world, allreduce=allreduce)
        import ctypes as C
        from fitre_b200 import _structs as S
        st = O.gradient(model, xs, ys, w, ncls, per, env=env)
        hv = O.hv(model, xs, w, ncls, per, st, v, env=env)
        info = S.KFAC_INFO()
        O.lib().ora_kfac_storage_indices(C.byref(model), C.byref(info))
        A, G = np.zeros(info.OmegaZSize), np.zeros(info.LambdaGSize)
        O.lib().ora_kfac_omega_z(C.byref(env), C.byref(model), xs, st.z, per, A, C.byref(info))
        O.lib().ora_kfac_lambda_delta(C.byref(env), C.byref(model), st.dx, per, G, C.byref(info))
        np.savez(out, loss=st.loss, gradient=st.gradient, hv=hv, A=A, G=G)
    else:
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world,
                                device_id=torch.device("cuda", rank))
        import gpu_util as G
        from fitre_b200 import api
        ctx = api.Context(rank)
        ctx.comm_init_from_torch()
        G._CTX["c"] = ctx
        import ctypes as C
        from fitre_b200 import _lib
        run = G.GpuRun(model, xs, ys, w, ncls, ref_softmax=1)
        hv = run.hv(v)
        info = api.computeKFACStorageIndices(model)
        scr = G.dev(np.zeros(_lib.load().fitre_kfac_mem_required(C.byref(model))))
        A, Gm = G.dev(np.zeros(info.OmegaZSize)), G.dev(np.zeros(info.LambdaGSize))
        api.computeOmegaZ(ctx, model, run.data, run.ws.z, per, A, info, scr)
        api.computeLambdaDelta(ctx, model, run.ws.dx, per, Gm, info, scr)
        # the factor inverses, divided among the ranks and exchanged
        info.regLambda, info.dampGamma = 1e-3, 1e-2
        Ai, Gi = G.dev(np.zeros(info.OmegaZSize)), G.dev(np.zeros(info.LambdaGSize))
        iscr = G.dev(np.zeros(_lib.load().fitre_kfac_invert_factors_mem_required(C.byref(model))))
        api.invertFactors(ctx, model, info, A, Ai, Gm, Gi, iscr)
        # natural gradient three ways: replicated inverses; factors owned by one rank per layer
        # (fused call, reduce onto the owner, only the natural gradient exchanged), explicit
        # inverses and Cholesky form
        L = _lib.load()
        nscr = G.dev(np.zeros(max(L.fitre_kfac_natural_gradient_mem_required(C.byref(model)),
                                  L.fitre_kfac_factors_and_inverses_mem_required(C.byref(model)))))
        ng_rep = G.dev(np.zeros(model.pSize))
        api.computeNaturalGradient(ctx, model, info, Ai, Gi, run.ws.gradient, ng_rep, nscr)
        ng_owned = {}
        ctx.set_kfac_distribution(1)
        for solver in (0, 1):
            ctx.set_kfac_solver(solver)
            A2, G2 = G.dev(np.zeros(info.OmegaZSize)), G.dev(np.zeros(info.LambdaGSize))
            Ai2, Gi2 = G.dev(np.zeros(info.OmegaZSize)), G.dev(np.zeros(info.LambdaGSize))
            api.computeFactorsAndInverses(ctx, model, run.data, run.ws.z, run.ws.dx, per, A2, Ai2, G2, Gi2,
                                          info, nscr)
            ng = G.dev(np.zeros(model.pSize))
            api.computeNaturalGradient(ctx, model, info, Ai2, Gi2, run.ws.gradient, ng, nscr)
            ng_owned[solver] = ng.cpu().numpy()
        ctx.set_kfac_solver(0)
        ctx.set_kfac_distribution(0)
        ng_rep = ng_rep.cpu().numpy()
        # the same gradient and Hv in the compensated tensor-core mode (sharded batch-norm statistics
        # and all-reduces around the tcgen05 kernels)
        g64, loss64 = run.gradient.copy(), run.loss
        del run
        ctx.set_precision(2)
        run3 = G.GpuRun(model, xs, ys, w, ncls, ref_softmax=1)
        hv3 = run3.hv(v)
        ctx.set_precision(0)
        # the host-buffer entry point on the shard: same bits as the device-resident calls (its
        # Hessian-vector slices travel to the host as each layer's all-reduce completes)
        g_host, hv_host = np.zeros(model.pSize), np.zeros(model.pSize)
        loss_host = api.gradientHvHost(ctx, model, xs, ys, w, v, per, ncls, 0.0, g_host, hv_host)
        # the same call with result buffers that are ONE shared, page-locked segment on all ranks:
        # every rank copies its share of each finished slice only, and finds the whole vectors
        P = model.pSize
        shm = "/dev/shm/fitre_mr_%s" % os.environ.get("MASTER_PORT", "0")
        if rank == 0:
            np.memmap(shm, dtype=np.float64, mode="w+", shape=(2 * P,)).flush()
        dist.barrier()
        buf = np.memmap(shm, dtype=np.float64, mode="r+", shape=(2 * P,))
        rt = torch.cuda.cudart()
        rt.cudaHostRegister(buf.ctypes.data, buf.nbytes, 0)
        ctx.set_host_results_shared(1)
        loss_shared = api.gradientHvHost(ctx, model, xs, ys, w, v, per, ncls, 0.0, buf[:P], buf[P:])
        g_shared, hv_shared = np.array(buf[:P]), np.array(buf[P:])
        # ... and with the replicated inputs (weights, direction) uploaded one chunk per rank and
        # all-gathered on the device
        dist.barrier()
        buf[:] = 0.0
        dist.barrier()
        ctx.set_host_inputs_replicated(1)
        loss_gathered = api.gradientHvHost(ctx, model, xs, ys, w, v, per, ncls, 0.0, buf[:P], buf[P:])
        ctx.set_host_inputs_replicated(0)
        ctx.set_host_results_shared(0)
        g_gathered, hv_gathered = np.array(buf[:P]), np.array(buf[P:])
        rt.cudaHostUnregister(buf.ctypes.data)
        dist.barrier()
        del buf
        if rank == 0:
            os.unlink(shm)
        np.savez(out, loss=loss64, gradient=g64, hv=hv, A=A.cpu().numpy(), peer_reduce=int(ctx.peer_reduce_enabled),
                 loss_shared=loss_shared, gradient_shared=g_shared, hv_shared=hv_shared,
                 loss_gathered=loss_gathered, gradient_gathered=g_gathered, hv_gathered=hv_gathered,
                 peer_launches=ctx.kernel_launches("peer_allreduce_kernel"),
                 loss_host=loss_host, gradient_host=g_host, hv_host=hv_host,
                 G=Gm.cpu().numpy(), Ainv=Ai.cpu().numpy(), Ginv=Gi.cpu().numpy(),
                 gradient_x3=run3.gradient, hv_x3=hv3, ng_rep=ng_rep, ng_owned=ng_owned[0],
                 ng_owned_chol=ng_owned[1])
        torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
