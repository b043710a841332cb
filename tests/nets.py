"""Small and full-size net descriptions shared by the tests (shapes follow the reference's
builders: nn/read_nn.c:500-725, nn/read_alexnet.c:14-243, nn/read_vgg.c:122-299)."""
from fitre_b200 import _structs as S


def test_vgg(batch, h=4, w=4, act=S.CNN_ACT_SOFTPLUS, bn=False, bias=True, classes=10):
    """readTestVGG (nn/read_vgg.c:122-212): conv3 2->3, conv3 3->4 + maxpool2, FC -> classes."""
    convs = [
        dict(cin=2, cout=3, h=h, w=w, k=3, pad=1, bn=bn, act=act, pool=None),
        dict(cin=3, cout=4, h=h, w=w, k=3, pad=1, bn=bn, act=act, pool=(S.MAX_POOL, 2, 2, 0)),
    ]
    fcs = [(4 * (h // 2) * (w // 2), classes, S.CNN_ACT_NONE)]
    return S.describe_model(convs, fcs, batch, bias)


def lenet_small(batch, act=S.CNN_ACT_SWISH, pool=S.AVG_POOL, bias=True, hw=16, classes=10, fc_act=None):
    """LeNet topology (conv5, pool2, conv5, pool2, 3 FC) on a 16x16 input; fc_act gives the two
    hidden FC layers their own activation (logistic / tanh of the reference's FC path)."""
    h1 = hw - 4
    h2 = h1 // 2 - 4
    convs = [
        dict(cin=3, cout=6, h=hw, w=hw, k=5, pad=0, bn=False, act=act, pool=(pool, 2, 2, 0)),
        dict(cin=6, cout=16, h=h1 // 2, w=h1 // 2, k=5, pad=0, bn=False, act=act, pool=(pool, 2, 2, 0)),
    ]
    fin = 16 * (h2 // 2) ** 2
    fa = act if fc_act is None else fc_act
    fcs = [(fin, 12, fa), (12, 11, fa), (11, classes, S.CNN_ACT_NONE)]
    return S.describe_model(convs, fcs, batch, bias)


def lenet(batch, act=S.CNN_ACT_SWISH, pool=S.AVG_POOL, bias=True):
    convs = [
        dict(cin=3, cout=6, h=32, w=32, k=5, pad=0, bn=False, act=act, pool=(pool, 2, 2, 0)),
        dict(cin=6, cout=16, h=14, w=14, k=5, pad=0, bn=False, act=act, pool=(pool, 2, 2, 0)),
    ]
    fcs = [(400, 120, act), (120, 84, act), (84, 10, S.CNN_ACT_NONE)]
    return S.describe_model(convs, fcs, batch, bias)


def alexnet_small(batch, act=S.CNN_ACT_SWISH, bn=True, bias=False, hw=8, ch=4, classes=10):
    """AlexNet-style: conv5 p2 + BN + act + maxpool3 s2 p1, twice, then 3 FC."""
    convs = [
        dict(cin=3, cout=ch, h=hw, w=hw, k=5, pad=2, bn=bn, act=act, pool=(S.MAX_POOL, 3, 2, 1)),
        dict(cin=ch, cout=ch, h=hw // 2, w=hw // 2, k=5, pad=2, bn=bn, act=act,
             pool=(S.MAX_POOL, 3, 2, 1)),
    ]
    fin = ch * (hw // 4) ** 2
    fcs = [(fin, 12, act), (12, 9, act), (9, classes, S.CNN_ACT_NONE)]
    return S.describe_model(convs, fcs, batch, bias)


def alexnet(batch, act=S.CNN_ACT_SWISH, bn=True, bias=False):
    convs = [
        dict(cin=3, cout=64, h=32, w=32, k=5, pad=2, bn=bn, act=act, pool=(S.MAX_POOL, 3, 2, 1)),
        dict(cin=64, cout=64, h=16, w=16, k=5, pad=2, bn=bn, act=act, pool=(S.MAX_POOL, 3, 2, 1)),
    ]
    fcs = [(4096, 384, act), (384, 192, act), (192, 10, S.CNN_ACT_NONE)]
    return S.describe_model(convs, fcs, batch, bias)


def vgg_small(batch, act=S.CNN_ACT_SWISH, bn=True, bias=False, hw=8, classes=10):
    """VGG-style: conv3 p1 + BN + act, pools after layers 0 and 2."""
    convs = [
        dict(cin=3, cout=8, h=hw, w=hw, k=3, pad=1, bn=bn, act=act, pool=(S.MAX_POOL, 2, 2, 0)),
        dict(cin=8, cout=8, h=hw // 2, w=hw // 2, k=3, pad=1, bn=bn, act=act, pool=None),
        dict(cin=8, cout=16, h=hw // 2, w=hw // 2, k=3, pad=1, bn=bn, act=act,
             pool=(S.MAX_POOL, 2, 2, 0)),
    ]
    fcs = [(16 * (hw // 4) ** 2, classes, S.CNN_ACT_NONE)]
    return S.describe_model(convs, fcs, batch, bias)


def vgg11(batch, act=S.CNN_ACT_SWISH, bn=True, bias=False, hw=32, classes=10, pool=S.MAX_POOL):
    chans = [(3, 64, True), (64, 128, True), (128, 256, False), (256, 256, True),
             (256, 512, False), (512, 512, True), (512, 512, False), (512, 512, True)]
    convs, s = [], hw
    for cin, cout, pooled in chans:
        convs.append(dict(cin=cin, cout=cout, h=s, w=s, k=3, pad=1, bn=bn, act=act,
                          pool=(pool, 2, 2, 0) if pooled else None))
        if pooled:
            s //= 2
    fcs = [(512 * s * s, classes, S.CNN_ACT_NONE)]
    return S.describe_model(convs, fcs, batch, bias)
