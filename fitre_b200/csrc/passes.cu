// Whole-network passes: forward, backward (gradient), R-forward, R-backward (Hessian-vector).
// They follow the reference's state contract -- every intermediate lands in `z`, the backward
// errors in `dx`, the R-forward values in `rz`, all with the offsets of CNN_MODEL -- so that a
// Hessian-vector call can consume what the gradient call left behind
// (functions/cnn_hessian_vec.cu:18-22).
// Reference: functions/cnn_forward.cu:48-382, cnn_backward.cu:76-857, cnn_hv_forward.cu:53-222,
// eval_convolution.cu:52-267,285-539, rop_fc_layer.cu:34-133, cnn_hv_backward.cu:70-912.
#include <algorithm>

#include "common.h"
#include "graphs.h"

namespace fitre {
namespace {

long align32(long n) { return (n + 31) / 32 * 32; }

long last_pool_elems(const CNN_MODEL *m) {
    const CONV_LAYER &c = m->convLayer[m->cLayers - 1];
    const POOL_LAYER &p = m->poolLayer[m->cLayers - 1];
    return (long)c.outChannels * p.outHeight * p.outWidth * m->batchSize;
}
long max_conv_volume(const CNN_MODEL *m) {
    long v = 0;
    for (int l = 0; l < m->cLayers; ++l)
        v = std::max(v, (long)m->convLayer[l].convVolumn * m->batchSize);
    return v;
}
long max_wgrad_scratch(const CNN_MODEL *m) {
    long v = 0;
    for (int l = 0; l < m->cLayers; ++l) {
        const CONV_LAYER &c = m->convLayer[l];
        v = std::max(v, conv_wgrad_scratch(m->batchSize, c.inChannels, c.height, c.width, c.kSize,
                                           c.padding, c.outChannels));
    }
    return v;
}
long max_weight_elems(const CNN_MODEL *m) {
    long v = 0;
    for (int l = 0; l < m->cLayers; ++l) {
        const CONV_LAYER &c = m->convLayer[l];
        v = std::max(v, (long)c.outChannels * c.inChannels * c.kSize * c.kSize);
    }
    return v;
}
long max_split_scratch(const CNN_MODEL *m) {
    long v = 0;
    for (int l = 0; l < m->cLayers; ++l) {
        const CONV_LAYER &c = m->convLayer[l];
        v = std::max(v, conv_fprop_scratch(m->batchSize, c.inChannels, c.height, c.width, c.kSize,
                                           c.padding, c.outChannels));
        if (l > 0)
            v = std::max(v, conv_dgrad_scratch(m->batchSize, c.inChannels, c.height, c.width,
                                               c.kSize, c.padding, c.outChannels));
    }
    return v;
}
long max_pool_map(const CNN_MODEL *m) {
    long v = 0;
    for (int l = 0; l < m->cLayers; ++l) v = std::max(v, pool_map_doubles(conv_geom(m, l), m->batchSize));
    return v;
}
long max_fc_elems(const CNN_MODEL *m) {
    long v = 0;
    for (int l = 0; l < m->lLayers; ++l)
        v = std::max(v, (long)std::max(m->fcLayer[l].in, m->fcLayer[l].out) * m->batchSize);
    return v;
}

// Data-parallel sweeps whose result is wanted on every rank (ctx->reduce_slices): the backward
// sweeps finish the parameter vector from its end towards its start, one layer at a time, so
// everything at or beyond `from` is final once the current layer's weight gradient is queued.
// That slice is all-reduced on the side communicator while the sweep computes the next layer.
void reduce_finished_slice(fitre_context *ctx, double *vec, long from) {
    if (!ctx->reduce_slices || ctx->world <= 1 || from >= ctx->reduced_from) return;
    comm_allreduce_async(ctx, vec + from, (size_t)(ctx->reduced_from - from));
    ctx->reduced_from = from;
}

const double *layer_input(const CNN_MODEL *m, const DEVICE_DATASET *data, const double *z, int l) {
    if (l == 0) return data->currentBatch;
    return z + m->zOffsets[l] + m->convLayer[l - 1].outputOffset;
}

}  // namespace

long forward_scratch(const CNN_MODEL *m) {
    return bn_scratch(0) + align32(last_pool_elems(m)) + align32(max_split_scratch(m));
}
long rop_forward_scratch(const CNN_MODEL *m) { return forward_scratch(m); }
long backward_scratch(const CNN_MODEL *m) {
    return bn_scratch(0) + align32(last_pool_elems(m)) + align32(max_wgrad_scratch(m)) +
           align32(max_weight_elems(m)) + align32(max_split_scratch(m)) + align32(max_pool_map(m));
}
long rop_backward_scratch(const CNN_MODEL *m) {
    return bn_scratch(0) + align32(last_pool_elems(m)) + align32(max_wgrad_scratch(m)) +
           2 * align32(max_weight_elems(m)) + align32(max_conv_volume(m)) +
           2 * align32(max_fc_elems(m)) + align32(max_split_scratch(m)) + align32(max_pool_map(m));
}

// ---------------------------------------------------------------------------------------------
double cnn_forward(fitre_context *ctx, const CNN_MODEL *m, const DEVICE_DATASET *data,
                   double *scratch, double *z, double *probs, double *errors, int n,
                   bool want_loss, bool running_stats) {
    const double *weights = data->weights;
    double *bnws = scratch;
    double *tmp = scratch + bn_scratch(0);
    double *split = tmp + align32(last_pool_elems(m));
    for (int l = 0; l < m->cLayers; ++l) {
        if (ctx->fwd_wait_event && l == ctx->fwd_wait_layer)
            FITRE_CUDA(cudaStreamWaitEvent(ctx->stream, ctx->fwd_wait_event, 0));
        const ConvGeom g = conv_geom(m, l);
        double *zl = z + g.zoff;
        ConvSeg seg{layer_input(m, data, z, l), weights + m->wOffsets[l]};
        conv_fprop(ctx, 1, &seg, m->bias ? weights + m->bOffsets[l] : nullptr, zl, n, g.Cin, g.H,
                   g.W, g.k, g.pad, g.Cout, split);
        conv_post_forward(ctx, g, n, zl, bnws, running_stats);
    }
    const ConvGeom lg = conv_geom(m, m->cLayers - 1);
    // the last convolution block's output is rewritten in the FC layout, as the reference does
    conv_to_fc(ctx, z + lg.zoff + lg.outOff, lg.Cout, n, lg.Hp, lg.Wp, tmp);
    long in_off = lg.zoff + lg.outOff;
    for (int l = 0; l < m->lLayers; ++l) {
        const FC_LAYER &f = m->fcLayer[l];
        double *out = z + m->zOffsets[m->cLayers + l + 1];
        dgemm(ctx, false, false, f.out, n, f.in, 1.0, weights + m->wOffsets[m->cLayers + l], f.out,
              z + in_off, f.in, 0.0, out + (long)f.out * n, f.out);
        if (m->bias) add_column_bias(ctx, out + (long)f.out * n, weights + m->bOffsets[m->cLayers + l], f.out, n);
        apply_activation(ctx, f.actFun, out + (long)f.out * n, out, (long)f.out * n);
        in_off = m->zOffsets[m->cLayers + l + 1];
    }
    const double *logits = z + m->zOffsets[m->cLayers + m->lLayers];
    const int classes = m->fcLayer[m->lLayers - 1].out;
    const double inv_ng = 1.0 / ((double)n * ctx->world);
    softmax_loss(ctx, logits, data->sampledTrainY, n, classes, probs, errors, inv_ng);
    if (!want_loss) return 0.0;
    comm_allreduce_small(ctx, ctx->dscal, 1);
    FITRE_CUDA(cudaMemcpyAsync(ctx->pinned, ctx->dscal, sizeof(double), cudaMemcpyDeviceToHost,
                               ctx->stream));
    stream_wait(ctx, ctx->stream);
    return ctx->pinned[0] * inv_ng;
}

// ---------------------------------------------------------------------------------------------
void cnn_backward(fitre_context *ctx, const CNN_MODEL *m, const DEVICE_DATASET *data,
                  double *scratch, double *z, double *gradient, double *dx, double *delta,
                  double *delta_new, int n) {
    const double *weights = data->weights;
    const int cL = m->cLayers, lL = m->lLayers;
    double *bnws = scratch;
    double *tmp = bnws + bn_scratch(0);
    double *wg = tmp + align32(last_pool_elems(m));
    double *wperm = wg + align32(max_wgrad_scratch(m));
    double *split = wperm + align32(max_weight_elems(m));
    unsigned char *pmap = max_pool_map(m) ? (unsigned char *)(split + align32(max_split_scratch(m))) : nullptr;
    const ConvGeom lg = conv_geom(m, cL - 1);

    for (int f = lL - 1; f >= 0; --f) {  // functions/cnn_backward.cu:111-280
        const FC_LAYER &l = m->fcLayer[f];
        const double *zl = z + m->zOffsets[cL + f + 1];
        act_backward(ctx, l.actFun, delta, zl + (long)l.out * n, zl, (long)l.out * n);
        const double *zin = (f == 0) ? z + lg.zoff + lg.outOff : z + m->zOffsets[cL + f];
        dgemm(ctx, false, true, l.out, l.in, n, 1.0, delta, l.out, zin, l.in, 0.0,
              gradient + m->wOffsets[cL + f], l.out);
        if (m->bias) row_sums(ctx, delta, l.out, n, gradient + m->bOffsets[cL + f]);
        vec_copy(ctx, (long)l.out * n, delta, dx + m->zOffsets[cL + f + 1]);
        dgemm(ctx, true, false, l.in, n, l.out, 1.0, weights + m->wOffsets[cL + f], l.out, delta,
              l.out, 0.0, delta_new, l.in);
        std::swap(delta, delta_new);
    }
    fc_to_conv(ctx, delta, lg.Cout, n, lg.Hp, lg.Wp, tmp);  // :310-326
    reduce_finished_slice(ctx, gradient, m->wOffsets[cL]);

    for (int c = cL - 1; c >= 0; --c) {  // :355-852
        const ConvGeom g = conv_geom(m, c);
        const double *zl = z + g.zoff;
        double *dxl = dx + g.zoff;
        const double *dconv = conv_post_backward(ctx, g, n, zl, dxl, delta,
                                                 m->bias ? gradient + m->bOffsets[c] : nullptr, bnws, pmap);
        ConvSeg wseg{layer_input(m, data, z, c), dconv};
        conv_wgrad(ctx, 1, &wseg, gradient + m->wOffsets[c], n, g.Cin, g.H, g.W, g.k, g.pad, g.Cout, wg);
        reduce_finished_slice(ctx, gradient, m->wOffsets[c]);
        if (c != 0) {
            ConvSeg dseg{dconv, weights + m->wOffsets[c]};
            conv_dgrad(ctx, 1, &dseg, delta_new, n, g.Cin, g.H, g.W, g.k, g.pad, g.Cout, wperm, split);
            std::swap(delta, delta_new);
        }
    }
}

// ---------------------------------------------------------------------------------------------
void cnn_rop_forward(fitre_context *ctx, const CNN_MODEL *m, const DEVICE_DATASET *data,
                     const double *z, const double *vector, double *rz, int n, double *scratch) {
    const double *weights = data->weights;
    double *bnws = scratch;
    double *tmp = scratch + bn_scratch(0);
    double *split = tmp + align32(last_pool_elems(m));
    for (int l = 0; l < m->cLayers; ++l) {
        const ConvGeom g = conv_geom(m, l);
        double *rzl = rz + g.zoff;
        // R{conv} = im2col(X) V + im2col(RX) W + Vb  (functions/eval_convolution.cu:339-381)
        ConvSeg segs[2];
        segs[0] = ConvSeg{layer_input(m, data, z, l), vector + m->wOffsets[l]};
        int nseg = 1;
        if (l > 0) {
            segs[1] = ConvSeg{rz + m->zOffsets[l] + m->convLayer[l - 1].outputOffset,
                              weights + m->wOffsets[l]};
            nseg = 2;
        }
        conv_fprop(ctx, nseg, segs, m->bias ? vector + m->bOffsets[l] : nullptr, rzl, n, g.Cin, g.H,
                   g.W, g.k, g.pad, g.Cout, split);
        conv_post_rop_forward(ctx, g, n, z + g.zoff, rzl, bnws);
    }
    const ConvGeom lg = conv_geom(m, m->cLayers - 1);
    conv_to_fc(ctx, rz + lg.zoff + lg.outOff, lg.Cout, n, lg.Hp, lg.Wp, tmp);
    long in_off = lg.zoff + lg.outOff;
    for (int l = 0; l < m->lLayers; ++l) {  // functions/rop_fc_layer.cu:34-133
        const FC_LAYER &f = m->fcLayer[l];
        const long cnt = (long)f.out * n;
        const double *z1 = z + m->zOffsets[m->cLayers + l + 1];
        double *out = rz + m->zOffsets[m->cLayers + l + 1];
        double *pre = out + cnt;
        dgemm(ctx, false, false, f.out, n, f.in, 1.0, vector + m->wOffsets[m->cLayers + l], f.out,
              z + in_off, f.in, 0.0, pre, f.out);
        dgemm(ctx, false, false, f.out, n, f.in, 1.0, weights + m->wOffsets[m->cLayers + l], f.out,
              rz + in_off, f.in, 1.0, pre, f.out);
        if (m->bias) add_column_bias(ctx, pre, vector + m->bOffsets[m->cLayers + l], f.out, n);
        vec_copy(ctx, cnt, pre, out);
        act_backward(ctx, f.actFun, out, z1 + cnt, z1, cnt);
        in_off = m->zOffsets[m->cLayers + l + 1];
    }
}

// ---------------------------------------------------------------------------------------------
// Host-buffer entry point only: everything of hv at or beyond `from` is final once the layers
// processed so far are done (the backward sweep runs from the last layer to the first) and, with
// ranks, their slice is all-reduced, so that slice goes to the host on the copy stream while the
// earlier layers are still computed.
static void send_finished_hv(fitre_context *ctx, const double *hv, long from, int slot) {
    if (!ctx->hv_host_dst || !ctx->copy_stream || from >= ctx->hv_sent_from) return;
    // with ranks the slice is final once its all-reduce on the side stream is done
    cudaStream_t after = ctx->stream;
    if (ctx->world > 1) {
        after = comm_async_stream(ctx);
        if (!after || !ctx->reduce_slices || ctx->reduced_from > from) return;
    }
    cudaEvent_t &ev = ctx->chunk_ev[slot % 24];
    if (!ev) FITRE_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
    FITRE_CUDA(cudaEventRecord(ev, after));
    FITRE_CUDA(cudaStreamWaitEvent(ctx->copy_stream, ev, 0));
    long lo, hi;
    host_share(ctx, from, ctx->hv_sent_from, lo, hi);
    if (hi > lo)
        FITRE_CUDA(cudaMemcpyAsync(ctx->hv_host_dst + lo, hv + lo, sizeof(double) * (size_t)(hi - lo),
                                   cudaMemcpyDeviceToHost, ctx->copy_stream));
    ctx->hv_sent_from = from;
}

void cnn_rop_backward(fitre_context *ctx, const CNN_MODEL *m, const DEVICE_DATASET *data,
                      const double *z, const double *dx, const double *lossErrors, double *rError,
                      const double *rz, const double *vector, double *hv, int n, double *scratch) {
    const double *weights = data->weights;
    const int cL = m->cLayers, lL = m->lLayers;
    double *bnws = scratch;
    double *tmp = bnws + bn_scratch(0);
    double *wg = tmp + align32(last_pool_elems(m));
    double *wperm = wg + align32(max_wgrad_scratch(m));
    double *rout = wperm + 2 * align32(max_weight_elems(m));
    double *t1 = rout + align32(max_conv_volume(m));
    double *t2 = t1 + align32(max_fc_elems(m));
    double *split = t2 + align32(max_fc_elems(m));
    unsigned char *pmap = max_pool_map(m) ? (unsigned char *)(split + align32(max_split_scratch(m))) : nullptr;
    const ConvGeom lg = conv_geom(m, cL - 1);

    for (int f = lL - 1; f >= 0; --f) {  // functions/cnn_hv_backward.cu:153-395
        const FC_LAYER &l = m->fcLayer[f];
        const long cnt = (long)l.out * n;
        const double *zl = z + m->zOffsets[cL + f + 1];
        const double *rzl = rz + m->zOffsets[cL + f + 1];
        const double *dxl = dx + m->zOffsets[cL + f + 1];
        if (l.actFun != FITRE_CNN_ACT_NONE && l.actFun != FITRE_ACT_LINEAR) {
            // errors that entered this activation in the backward pass
            const double *din = lossErrors;
            if (f != lL - 1) {
                const FC_LAYER &ll = m->fcLayer[f + 1];
                dgemm(ctx, true, false, ll.in, n, ll.out, 1.0, weights + m->wOffsets[cL + f + 1],
                      ll.out, dx + m->zOffsets[cL + f + 2], ll.out, 0.0, t1, ll.in);
                din = t1;
            }
            act_rop_backward(ctx, l.actFun, rError, din, rzl + cnt, zl + cnt, zl, cnt);
        }
        const double *zin = (f == 0) ? z + lg.zoff + lg.outOff : z + m->zOffsets[cL + f];
        const double *rzin = (f == 0) ? rz + lg.zoff + lg.outOff : rz + m->zOffsets[cL + f];
        double *hw = hv + m->wOffsets[cL + f];
        dgemm(ctx, false, true, l.out, l.in, n, 1.0, rError, l.out, zin, l.in, 0.0, hw, l.out);
        dgemm(ctx, false, true, l.out, l.in, n, 1.0, dxl, l.out, rzin, l.in, 1.0, hw, l.out);
        if (m->bias) row_sums(ctx, rError, l.out, n, hv + m->bOffsets[cL + f]);
        dgemm(ctx, true, false, l.in, n, l.out, 1.0, weights + m->wOffsets[cL + f], l.out, rError,
              l.out, 0.0, t2, l.in);
        dgemm(ctx, true, false, l.in, n, l.out, 1.0, vector + m->wOffsets[cL + f], l.out, dxl,
              l.out, 1.0, t2, l.in);
        vec_copy(ctx, (long)l.in * n, t2, rError);
    }
    fc_to_conv(ctx, rError, lg.Cout, n, lg.Hp, lg.Wp, tmp);  // :414-427
    reduce_finished_slice(ctx, hv, m->wOffsets[cL]);
    send_finished_hv(ctx, hv, m->wOffsets[cL], cL);

    for (int c = cL - 1; c >= 0; --c) {  // :436-907
        const ConvGeom g = conv_geom(m, c);
        const double *zl = z + g.zoff, *rzl = rz + g.zoff, *dxl = dx + g.zoff;
        conv_post_rop_backward(ctx, g, n, zl, rzl, dxl, rError, rout,
                               m->bias ? hv + m->bOffsets[c] : nullptr, bnws, pmap);
        const double *dprev = g.bn ? dxl + g.bnOff : dxl + g.actOff;
        // R dW = im2col(X)' Rdelta + im2col(RX)' delta  (:727-803)
        ConvSeg ws[2];
        ws[0] = ConvSeg{layer_input(m, data, z, c), rout};
        int nseg = 1;
        if (c != 0) {
            ws[1] = ConvSeg{rz + m->zOffsets[c] + m->convLayer[c - 1].outputOffset, dprev};
            nseg = 2;
        }
        conv_wgrad(ctx, nseg, ws, hv + m->wOffsets[c], n, g.Cin, g.H, g.W, g.k, g.pad, g.Cout, wg);
        reduce_finished_slice(ctx, hv, m->wOffsets[c]);
        if (c != 0) {  // Rdelta <- dgrad(Rdelta, W) + dgrad(delta, V)  (:854-898)
            ConvSeg ds[2] = {ConvSeg{rout, weights + m->wOffsets[c]},
                             ConvSeg{dprev, vector + m->wOffsets[c]}};
            conv_dgrad(ctx, 2, ds, rError, n, g.Cin, g.H, g.W, g.k, g.pad, g.Cout, wperm, split);
        }
        send_finished_hv(ctx, hv, m->wOffsets[c], c);
    }
}

namespace {
// A pass may be replayed from a captured graph where launch latency is what it costs (small nets:
// a LeNet Hessian-vector product is ~120 dependent kernels of a few microseconds each) and nothing
// in it depends on the host: one rank (no collectives), fp64 kernels (the tensor-core modes grow
// their staging buffer on demand), no host-buffer streaming hooks, no event timing.
bool pass_graphable(const fitre_context *ctx) {
    return ctx->use_graphs && ctx->use_pass_graphs && ctx->world == 1 && !ctx->prof_on &&
           ctx->precision == FITRE_PRECISION_FP64 && !ctx->hv_host_dst && !ctx->fwd_wait_event;
}
long long model_key(const CNN_MODEL *m) {  // FNV-1a over the model description
    const unsigned char *b = reinterpret_cast<const unsigned char *>(m);
    unsigned long long h = 1469598103934665603ull;
    for (size_t i = 0; i < sizeof(CNN_MODEL); ++i) h = (h ^ b[i]) * 1099511628211ull;
    return (long long)h;
}
// the graph of `key` among the few kept, or the slot that is overwritten next
fitre_context::CapturedGraph &pick_graph(fitre_context::CapturedGraph *slots, int count, int &next,
                                         const std::vector<long long> &key) {
    for (int i = 0; i < count; ++i)
        if (slots[i].exec && slots[i].key == key) return slots[i];
    fitre_context::CapturedGraph &g = slots[next];
    next = (next + 1) % count;
    return g;
}
void cnn_hv_direct(fitre_context *ctx, const CNN_MODEL *m, const DEVICE_DATASET *data, const double *z,
                   const double *probs, const double *lossErrors, const double *dx, const double *vector,
                   double *hv, int n, double *devPtr);
}  // namespace

void cnn_hv(fitre_context *ctx, const CNN_MODEL *m, const DEVICE_DATASET *data, const double *z,
            const double *probs, const double *lossErrors, const double *dx, const double *vector,
            double *hv, int n, double *devPtr) {
    if (!pass_graphable(ctx)) {
        cnn_hv_direct(ctx, m, data, z, probs, lossErrors, dx, vector, hv, n, devPtr);
        return;
    }
    const std::vector<long long> key = {model_key(m), ptr_key(data->weights), ptr_key(data->currentBatch), ptr_key(z),
                                        ptr_key(probs), ptr_key(lossErrors), ptr_key(dx), ptr_key(vector),
                                        ptr_key(hv), ptr_key(devPtr), n, ctx->ref_softmax, ctx->use_tma};
    run_graphed(ctx, pick_graph(ctx->graph_hv, 4, ctx->graph_hv_next, key), key,
                [&] { cnn_hv_direct(ctx, m, data, z, probs, lossErrors, dx, vector, hv, n, devPtr); },
                &ctx->use_pass_graphs);
}

namespace {
void cnn_gradient_direct(fitre_context *ctx, const CNN_MODEL *m, const DEVICE_DATASET *data, double *ws,
                         double *z, double *dx, double *probs, double *lossErrors, double *gradient,
                         double *errors, double *errors1, int n, double weightDecay) {
    cnn_forward(ctx, m, data, ws, z, probs, lossErrors, n, false);
    const int classes = m->fcLayer[m->lLayers - 1].out;
    vec_copy(ctx, (long)classes * n, lossErrors, errors);
    // the gradient is a batch sum: each layer's slice is all-reduced as soon as the backward
    // sweep has finished it, on the side communicator, under the rest of the sweep
    ctx->reduce_slices = true;
    ctx->reduced_from = m->pSize;
    try {
        cnn_backward(ctx, m, data, ws, z, gradient, dx, errors, errors1, n);
    } catch (...) {
        ctx->reduce_slices = false;
        throw;
    }
    ctx->reduce_slices = false;
    comm_async_join(ctx);
    vec_axpy(ctx, m->pSize, weightDecay, data->weights, gradient);
}
}  // namespace

void cnn_gradient(fitre_context *ctx, const CNN_MODEL *m, const DEVICE_DATASET *data, double *ws, double *z,
                  double *dx, double *probs, double *lossErrors, double *gradient, double *errors,
                  double *errors1, int n, double weightDecay) {
    if (!pass_graphable(ctx)) {
        cnn_gradient_direct(ctx, m, data, ws, z, dx, probs, lossErrors, gradient, errors, errors1, n, weightDecay);
        return;
    }
    const std::vector<long long> key = {model_key(m), ptr_key(data->weights), ptr_key(data->currentBatch),
                                        ptr_key(data->sampledTrainY), ptr_key(ws), ptr_key(z), ptr_key(dx),
                                        ptr_key(probs), ptr_key(lossErrors), ptr_key(gradient), ptr_key(errors),
                                        ptr_key(errors1), n, bits_key(weightDecay), ctx->ref_softmax, ctx->use_tma};
    run_graphed(ctx, pick_graph(ctx->graph_grad, 2, ctx->graph_grad_next, key), key, [&] {
        cnn_gradient_direct(ctx, m, data, ws, z, dx, probs, lossErrors, gradient, errors, errors1, n, weightDecay);
    }, &ctx->use_pass_graphs);
}

namespace {
// functions/cnn_hessian_vec.cu:18-122: devPtr = [rz (zSize) | rError (maxDelta) | scratch]
void cnn_hv_direct(fitre_context *ctx, const CNN_MODEL *m, const DEVICE_DATASET *data, const double *z,
                   const double *probs, const double *lossErrors, const double *dx, const double *vector,
                   double *hv, int n, double *devPtr) {
    double *rz = devPtr;
    double *rError = rz + align32(m->zSize);
    double *scratch = rError + align32(max_delta_elems(m));
    cnn_rop_forward(ctx, m, data, z, vector, rz, n, scratch);
    const int classes = m->fcLayer[m->lLayers - 1].out;
    const double inv_ng = 1.0 / ((double)n * ctx->world);
    softmax_rop_error(ctx, rz + m->zOffsets[m->cLayers + m->lLayers], probs, n, classes, rError,
                      inv_ng);
    // hv is a batch sum: every layer's slice is all-reduced as soon as the sweep has finished it
    ctx->reduce_slices = true;
    ctx->reduced_from = m->pSize;
    try {
        cnn_rop_backward(ctx, m, data, z, dx, lossErrors, rError, rz, vector, hv, n, scratch);
    } catch (...) {
        ctx->reduce_slices = false;
        throw;
    }
    ctx->reduce_slices = false;
    comm_async_join(ctx);
}
}  // namespace

}  // namespace fitre
