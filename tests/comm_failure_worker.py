"""Child process of tests/test_gpu_failure_paths.py: one failure scenario of the data-parallel
plumbing per run, result printed as one JSON line.  The failures are made on the host (a peer
that never joins, an error code from a stand-in NCCL library, a stream parked in a host
function); nothing here makes a GPU wait, spin or fault."""
import ctypes as C
import json
import os
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, HERE)


def small_case():
    import gpu_util as G
    import nets
    model = nets.vgg_small(4)
    from fitre_b200 import api
    api.finalize(model)
    x, y, w, v, ncls = G.synth(model, 4, seed=3)
    return model, x, y, w, v, ncls


def gradient_status(ctx, model, x, y, w, ncls):
    """status of one fitre_compute_cnn_gradient call (0 = OK) and the seconds it took"""
    import gpu_util as G
    from fitre_b200 import api
    ws = api.Workspace(model, ncls)
    data = api.make_dataset(G.dev(w), G.dev(x), G.dev(y), ncls)
    t0 = time.time()
    try:
        api.computeCNNGradient(ctx, model, data, ws.scratch, ws.z, ws.dx, ws.probs, ws.errors, ws.gradient,
                               0, model.batchSize, 0.0)
        return 0, time.time() - t0, ""
    except api.FitreError as e:
        return e.status, time.time() - t0, str(e)


def main():
    mode = sys.argv[1]
    import torch
    torch.cuda.set_device(0)
    from fitre_b200 import api
    ctx = api.Context(0)
    out = {"mode": mode}
    if mode in ("fake_init_never_returns", "real_peer_never_joins"):
        ctx.set_comm_timeout(2.0)
        uid = api.Context.comm_unique_id()
        t0 = time.time()
        try:
            ctx.comm_init(uid, 0, 2)      # rank 1 does not exist
            out["status"] = 0
        except api.FitreError as e:
            out["status"], out["text"] = e.status, str(e)
        out["seconds"] = time.time() - t0
        out["world_after"] = ctx.world
        model, x, y, w, v, ncls = small_case()
        out["single_gpu_status_after"] = gradient_status(ctx, model, x, y, w, ncls)[0]
    elif mode in ("fake_async_error", "fake_stalled_collective"):
        ctx.set_comm_timeout(1.0 if mode == "fake_stalled_collective" else 30.0)
        ctx.comm_init(api.Context.comm_unique_id(), 0, 2)
        out["world"] = ctx.world
        model, x, y, w, v, ncls = small_case()
        out["status"], out["seconds"], out["text"] = gradient_status(ctx, model, x, y, w, ncls)
        out["status_again"] = gradient_status(ctx, model, x, y, w, ncls)[0]   # aborted: fails fast
        fake = C.CDLL(os.environ["FITRE_NCCL_LIBRARY"])
        out["aborts"], out["destroys"] = fake.fake_nccl_count(0), fake.fake_nccl_count(1)
        time.sleep(float(os.environ.get("FAKE_NCCL_STALL_MS", "0")) / 1000.0 * 3)  # let parked host functions end
        ctx.comm_init(api.Context.comm_unique_id(), 0, 1)                     # back to one GPU
        out["single_gpu_status_after"] = gradient_status(ctx, model, x, y, w, ncls)[0]
    print(json.dumps(out), flush=True)
    os._exit(0)   # a set-up thread may still sit in the library: do not wait for it


if __name__ == "__main__":
    main()
