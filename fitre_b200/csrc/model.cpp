// Model description: builders, derived offsets and sizes, validation.
// Reference: nn/utils.c:12-172 (sizes and offset tables), nn/read_vgg.c:25-120 (per-layer
// z layout), nn/read_nn.c:500-725 (LeNet), nn/read_alexnet.c:14-243, nn/read_vgg.c:122-299.
#include <climits>
#include <cmath>
#include <cstring>

#include "common.h"

namespace {

struct Cursor {  // running 64-bit offset that refuses to leave the int range of the ABI structs
    long v = 0;
    bool overflow = false;
    int take(long n) {
        long at = v;
        v += n;
        if (v > INT_MAX) overflow = true;
        return overflow ? 0 : (int)at;
    }
};

int pooled(int in, int ks, int stride, int pad) {  // functions/dev_pool.cu:226-227
    return (int)std::floor((double)(in - ks + 2 * pad) / (double)stride + 1.0);
}

void set_conv(CNN_MODEL *m, int l, int cin, int cout, int h, int w, int k, int pad, int bn,
              int act, int poolType, int pk, int ps, int pp) {
    CONV_LAYER &c = m->convLayer[l];
    c.inChannels = cin;
    c.outChannels = cout;
    c.height = h;
    c.width = w;
    c.kSize = k;
    c.stride = 1;
    c.padding = pad;
    c.batchNorm = bn ? FITRE_BATCH_NORM : FITRE_NO_BATCH_NORM;
    m->actFuns[l] = act;
    POOL_LAYER &p = m->poolLayer[l];
    p.type = poolType;
    p.pSize = pk;
    p.stride = ps;
    p.padding = pp;
}

void set_fc(CNN_MODEL *m, int l, int in, int out, int act) {
    m->fcLayer[l].in = in;
    m->fcLayer[l].out = out;
    m->fcLayer[l].actFun = act;
    m->fcLayer[l].batchNorm = 0;
}

bool act_supported(int a) {
    return a == FITRE_CNN_ACT_NONE || a == FITRE_ACT_LINEAR || a == FITRE_CNN_ACT_SOFTPLUS ||
           a == FITRE_CNN_ACT_RELU || a == FITRE_CNN_ACT_SWISH || a == FITRE_ACT_LOGISTIC ||
           a == FITRE_ACT_TANH;
}

}  // namespace

extern "C" int fitre_model_finalize(CNN_MODEL *m) {
    if (!m || m->cLayers < 1 || m->lLayers < 0 || m->batchSize < 1 ||
        m->cLayers + m->lLayers + 2 > FITRE_MAX_LAYERS)
        return FITRE_ERR_BAD_ARG;
    const long B = m->batchSize;
    const int L = m->cLayers + m->lLayers;

    // per-layer geometry and the in-block offsets of z (conv | bn | stats | act | pool)
    for (int l = 0; l < m->cLayers; ++l) {
        CONV_LAYER &c = m->convLayer[l];
        POOL_LAYER &p = m->poolLayer[l];
        if (c.stride < 1 || c.kSize < 1) return FITRE_ERR_BAD_ARG;
        c.outHeight = (c.height + 2 * c.padding - c.kSize) / c.stride + 1;
        c.outWidth = (c.width + 2 * c.padding - c.kSize) / c.stride + 1;
        p.height = c.outHeight;
        p.width = c.outWidth;
        const bool has_pool = p.type != FITRE_NO_POOL;
        p.outHeight = has_pool ? pooled(p.height, p.pSize, p.stride, p.padding) : p.height;
        p.outWidth = has_pool ? pooled(p.width, p.pSize, p.stride, p.padding) : p.width;
        const long vol = (long)c.outHeight * c.outWidth * c.outChannels;
        const long V = vol * B;
        Cursor cur;
        cur.take(V);  // convolution output sits at 0
        const bool bn = c.batchNorm != FITRE_NO_BATCH_NORM;
        if (bn) {
            c.batchNormOffset = cur.take(V);
            c.meansOffset = (int)std::min<long>(V, INT_MAX);  // relative to the BN output
            c.variancesOffset = c.meansOffset + c.outChannels;
            c.runningMeansOffset = c.variancesOffset + c.outChannels;
            c.runningVariancesOffset = c.runningMeansOffset + c.outChannels;
            cur.take(4L * c.outChannels);
        } else {
            c.batchNormOffset = c.meansOffset = c.variancesOffset = INT_MAX;
            c.runningMeansOffset = c.runningVariancesOffset = INT_MAX;
        }
        c.activationOffset = cur.take(V);
        if (has_pool) {
            c.poolOffset = cur.take((long)p.outHeight * p.outWidth * c.outChannels * B);
            c.outputOffset = c.poolOffset;
        } else {
            c.poolOffset = INT_MAX;
            c.outputOffset = c.activationOffset;
        }
        if (cur.overflow) return FITRE_ERR_TOO_LARGE;
        c.convVolumn = (int)vol;
        c.activationVolumn = (int)vol;
        c.batchNormVolumn = bn ? INT_MAX : (int)vol;
        c.poolVolumn = has_pool ? p.outHeight * p.outWidth * c.outChannels : INT_MAX;
    }
    for (int l = 0; l < m->lLayers; ++l) {
        if ((long)m->fcLayer[l].out * B > INT_MAX) return FITRE_ERR_TOO_LARGE;
        m->fcLayer[l].offset = (int)(m->fcLayer[l].out * B);
    }

    // flat parameter vector: [W_0 (b_0) W_1 (b_1) ...], convolutions first
    std::memset(m->wOffsets, 0, sizeof(m->wOffsets));
    std::memset(m->bOffsets, 0, sizeof(m->bOffsets));
    Cursor pc;
    for (int i = 0; i < L; ++i) {
        long wsz, bsz;
        if (i < m->cLayers) {
            const CONV_LAYER &c = m->convLayer[i];
            wsz = (long)c.outChannels * c.inChannels * c.kSize * c.kSize;
            bsz = c.outChannels;
        } else {
            const FC_LAYER &f = m->fcLayer[i - m->cLayers];
            wsz = (long)f.out * f.in;
            bsz = f.out;
        }
        m->wOffsets[i] = pc.take(wsz);
        m->bOffsets[i] = m->bias ? pc.take(bsz) : INT_MAX;
    }
    if (pc.overflow) return FITRE_ERR_TOO_LARGE;
    if (!m->bias) m->wOffsets[L] = (int)pc.v;
    m->pSize = (int)pc.v;

    // z blocks: index l+1 holds layer l; zOffsets[0] = zOffsets[1] = 0
    std::memset(m->zOffsets, 0, sizeof(m->zOffsets));
    std::memset(m->zztOffsets, 0, sizeof(m->zztOffsets));
    Cursor zc, zzt;
    long maxBlock = 0;
    for (int i = 0; i < L; ++i) {
        long block, outs;
        if (i < m->cLayers) {
            const CONV_LAYER &c = m->convLayer[i];
            const POOL_LAYER &p = m->poolLayer[i];
            const long V = (long)c.convVolumn * B;
            block = 2 * V;
            if (c.batchNorm != FITRE_NO_BATCH_NORM) block += V + 4L * c.outChannels;
            if (p.type != FITRE_NO_POOL) block += (long)c.poolVolumn * B;
            outs = V;
        } else {
            block = 2L * m->fcLayer[i - m->cLayers].out * B;  // activation + pre-activation
            outs = (long)m->fcLayer[i - m->cLayers].out * B;
        }
        m->zOffsets[i + 1] = zc.take(block);
        m->zztOffsets[i + 1] = zzt.take(outs);
        if (block > maxBlock) maxBlock = block;
    }
    if (zc.overflow) return FITRE_ERR_TOO_LARGE;
    m->zOffsets[L + 1] = (int)zc.v;
    m->zztOffsets[L + 1] = (int)zzt.v;
    m->zSize = (int)zc.v;
    m->zztSize = (int)zzt.v;
    m->maxDeltaSize = (int)maxBlock;
    return FITRE_OK;
}

extern "C" int fitre_model_validate(const CNN_MODEL *m) {
    if (!m || m->cLayers < 1 || m->batchSize < 1) return FITRE_ERR_BAD_ARG;
    for (int l = 0; l < m->cLayers; ++l) {
        const CONV_LAYER &c = m->convLayer[l];
        const POOL_LAYER &p = m->poolLayer[l];
        if (c.stride != 1) return FITRE_ERR_UNSUPPORTED;  // dgrad is stride-1 only (dev_backprop_convolution.cu:173-177)
        if (c.kSize > 7 || c.padding >= c.kSize) return FITRE_ERR_UNSUPPORTED;
        if (!act_supported(m->actFuns[l])) return FITRE_ERR_UNSUPPORTED;
        if (c.batchNorm != FITRE_NO_BATCH_NORM && c.batchNorm != FITRE_BATCH_NORM)
            return FITRE_ERR_UNSUPPORTED;
        if (l > 0) {
            const CONV_LAYER &q = m->convLayer[l - 1];
            const POOL_LAYER &pp = m->poolLayer[l - 1];
            if (c.inChannels != q.outChannels || c.height != pp.outHeight || c.width != pp.outWidth)
                return FITRE_ERR_BAD_ARG;
        }
        if (p.type == FITRE_MAX_POOL || p.type == FITRE_AVG_POOL) {
            // the reference's window start (k-1)s + ksize - 2p equals k*s - p only then
            if (p.pSize - p.stride != p.padding) return FITRE_ERR_UNSUPPORTED;
            if (p.pSize > 4) return FITRE_ERR_UNSUPPORTED;
            if (p.type == FITRE_AVG_POOL &&
                (p.padding != 0 || p.stride != p.pSize || c.outHeight != c.outWidth ||
                 c.outHeight % p.pSize != 0))
                return FITRE_ERR_UNSUPPORTED;  // dev_pool.cu:269-298 handles only this form
        } else if (p.type != FITRE_NO_POOL) {
            return FITRE_ERR_UNSUPPORTED;
        }
    }
    const POOL_LAYER &lp = m->poolLayer[m->cLayers - 1];
    if (lp.outHeight != lp.outWidth) return FITRE_ERR_UNSUPPORTED;  // dev_transpose.cu:26-28
    if (m->lLayers < 1) return FITRE_ERR_UNSUPPORTED;
    const CONV_LAYER &lc = m->convLayer[m->cLayers - 1];
    if (m->fcLayer[0].in != lc.outChannels * lp.outHeight * lp.outWidth) return FITRE_ERR_BAD_ARG;
    for (int l = 0; l < m->lLayers; ++l) {
        if (!act_supported(m->fcLayer[l].actFun)) return FITRE_ERR_UNSUPPORTED;
        if (l > 0 && m->fcLayer[l].in != m->fcLayer[l - 1].out) return FITRE_ERR_BAD_ARG;
    }
    return FITRE_OK;
}

extern "C" int fitre_read_lenet_cnn(CNN_MODEL *m, int channels, int width, int height,
                                    int batchSize, int enableBias, int enableBatchNorm,
                                    int actFun, int poolType) {
    if (!m) return FITRE_ERR_BAD_ARG;
    std::memset(m, 0, sizeof(*m));
    set_conv(m, 0, channels, 6, height, width, 5, 0, enableBatchNorm, actFun, poolType, 2, 2, 0);
    const int h1 = (height - 4) / 2, w1 = (width - 4) / 2;
    set_conv(m, 1, 6, 16, h1, w1, 5, 0, enableBatchNorm, actFun, poolType, 2, 2, 0);
    const int h2 = (h1 - 4) / 2, w2 = (w1 - 4) / 2;
    m->cLayers = 2;
    set_fc(m, 0, 16 * h2 * w2, 120, actFun);
    set_fc(m, 1, 120, 84, actFun);
    set_fc(m, 2, 84, 10, FITRE_CNN_ACT_NONE);
    m->lLayers = 3;
    m->name = FITRE_NET_LENET;
    m->bias = enableBias;
    m->enableBatchNorm = enableBatchNorm;
    m->batchSize = batchSize;
    return fitre_model_finalize(m);
}

extern "C" int fitre_read_alexnet_cnn(CNN_MODEL *m, int batchSize, int height, int width,
                                      int numClasses, int enableBias, int enableBatchNorm,
                                      int actFun) {
    if (!m) return FITRE_ERR_BAD_ARG;
    std::memset(m, 0, sizeof(*m));
    set_conv(m, 0, 3, 64, height, width, 5, 2, enableBatchNorm, actFun, FITRE_MAX_POOL, 3, 2, 1);
    const int h1 = pooled(height, 3, 2, 1), w1 = pooled(width, 3, 2, 1);
    set_conv(m, 1, 64, 64, h1, w1, 5, 2, enableBatchNorm, actFun, FITRE_MAX_POOL, 3, 2, 1);
    const int h2 = pooled(h1, 3, 2, 1), w2 = pooled(w1, 3, 2, 1);
    m->cLayers = 2;
    set_fc(m, 0, 64 * h2 * w2, 384, actFun);
    set_fc(m, 1, 384, 192, actFun);
    set_fc(m, 2, 192, numClasses, FITRE_CNN_ACT_NONE);
    m->lLayers = 3;
    m->name = FITRE_NET_ALEXNET;
    m->bias = enableBias;
    m->enableBatchNorm = enableBatchNorm;
    m->batchSize = batchSize;
    return fitre_model_finalize(m);
}

extern "C" int fitre_read_vgg11(CNN_MODEL *m, int batchSize, int height, int width,
                                int numClasses, int inChannels, int enableBias,
                                int enableBatchNorm, int actFun) {
    if (!m) return FITRE_ERR_BAD_ARG;
    std::memset(m, 0, sizeof(*m));
    static const int chans[8] = {64, 128, 256, 256, 512, 512, 512, 512};
    static const int pool_after[8] = {1, 1, 0, 1, 0, 1, 0, 1};
    int h = height, w = width, cin = inChannels;
    for (int l = 0; l < 8; ++l) {
        set_conv(m, l, cin, chans[l], h, w, 3, 1, enableBatchNorm, actFun,
                 pool_after[l] ? FITRE_MAX_POOL : FITRE_NO_POOL, 2, 2, 0);
        if (pool_after[l]) {
            h /= 2;
            w /= 2;
        }
        cin = chans[l];
    }
    m->cLayers = 8;
    set_fc(m, 0, 512 * h * w, numClasses, FITRE_CNN_ACT_NONE);
    m->lLayers = 1;
    m->name = FITRE_NET_VGG11;
    m->bias = enableBias;
    m->enableBatchNorm = enableBatchNorm;
    m->batchSize = batchSize;
    return fitre_model_finalize(m);
}

extern "C" int fitre_read_test_vgg(CNN_MODEL *m, int batchSize, int height, int width,
                                   int numClasses, int inChannels, int enableBias, int batchNorm,
                                   int actFun) {
    if (!m) return FITRE_ERR_BAD_ARG;
    std::memset(m, 0, sizeof(*m));
    set_conv(m, 0, inChannels, 3, height, width, 3, 1, batchNorm, actFun, FITRE_NO_POOL, 2, 2, 0);
    set_conv(m, 1, 3, 4, height, width, 3, 1, batchNorm, actFun, FITRE_MAX_POOL, 2, 2, 0);
    m->cLayers = 2;
    set_fc(m, 0, 4 * (height / 2) * (width / 2), numClasses, FITRE_CNN_ACT_NONE);
    m->lLayers = 1;
    m->bias = enableBias;
    m->enableBatchNorm = batchNorm;
    m->batchSize = batchSize;
    return fitre_model_finalize(m);
}

namespace fitre {

ConvGeom conv_geom(const CNN_MODEL *m, int l) {
    const CONV_LAYER &c = m->convLayer[l];
    const POOL_LAYER &p = m->poolLayer[l];
    ConvGeom g;
    g.Cin = c.inChannels;
    g.Cout = c.outChannels;
    g.H = c.height;
    g.W = c.width;
    g.Ho = c.outHeight;
    g.Wo = c.outWidth;
    g.k = c.kSize;
    g.pad = c.padding;
    g.bn = c.batchNorm != FITRE_NO_BATCH_NORM;
    g.act = m->actFuns[l];
    g.poolType = p.type;
    g.pk = p.pSize;
    g.ps = p.stride;
    g.pp = p.padding;
    g.Hp = p.outHeight;
    g.Wp = p.outWidth;
    g.zoff = m->zOffsets[l + 1];
    g.actOff = c.activationOffset;
    g.poolOff = c.poolOffset;
    g.bnOff = c.batchNormOffset;
    g.outOff = c.outputOffset;
    g.meanOff = c.meansOffset;
    g.varOff = c.variancesOffset;
    return g;
}

void model_check_batch(const CNN_MODEL *m, int curBatchSize) {
    FITRE_REQUIRE(m != nullptr, FITRE_ERR_BAD_ARG, "model is NULL");
    // z offsets are laid out for model->batchSize; the FC pre-activation copy sits at
    // out*curBatchSize (functions/eval_gradient.cu:137): only full batches are consistent.
    FITRE_REQUIRE(curBatchSize == m->batchSize, FITRE_ERR_BAD_ARG,
                  "curBatchSize must equal model->batchSize");
    int rc = fitre_model_validate(m);
    FITRE_REQUIRE(rc == FITRE_OK, rc, "model outside the supported path");
}

long max_delta_elems(const CNN_MODEL *m) {
    long md = m->maxDeltaSize;
    for (int l = 0; l < m->cLayers; ++l) {
        const CONV_LAYER &c = m->convLayer[l];
        long v = (long)m->batchSize * c.height * c.width * c.inChannels;
        if (v > md) md = v;
    }
    for (int l = 0; l < m->lLayers; ++l) {
        long v = (long)m->batchSize * std::max(m->fcLayer[l].in, m->fcLayer[l].out);
        if (v > md) md = v;
    }
    return md;
}

}  // namespace fitre
