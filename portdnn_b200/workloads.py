"""Layer tables of the benchmark networks, as sequences of portDNN operator calls.

The reference has no network runner beyond its samples (tools/layer.h, tools/network.h: a list of
layers run one after another); its benchmarks time layers from tables such as
bench/conv2d/resnet_params.def and bench/conv2d/vgg_params.def.  The tables here are built the same
way (one Conv2DParams per layer via helpers::add_padding_to) for the shapes the workload
configurations name.
"""
from . import api


class ConvLayer:
    """One convolution followed by bias + ReLU, as tools/layer.h chains ConvolutionLayer,
    BiasAddLayer and ActivationLayer."""

    def __init__(self, name, params, src, dst, activation=api.ACT_RELU):
        self.name, self.params, self.src, self.dst, self.activation = name, params, src, dst, activation

    @property
    def flops(self):
        # forward counter of the reference's benchmarks, bench/conv2d/base_convolution_fixture.h:85-88
        p = self.params
        return 2 * p.batch * p.out_rows * p.out_cols * p.window_rows * p.window_cols * p.channels * p.features

    @property
    def ideal_bytes(self, elem=2):
        p = self.params
        return elem * (p.batch * p.in_rows * p.in_cols * p.channels + p.window_rows * p.window_cols * p.channels *
                       p.features + p.batch * p.out_rows * p.out_cols * p.features)


class PoolLayer:
    def __init__(self, name, op, params, src, dst):
        self.name, self.op, self.params, self.src, self.dst = name, op, params, src, dst

    @property
    def ideal_bytes(self, elem=2):
        p = self.params
        return elem * p.batch * p.channels * (p.in_rows * p.in_cols + p.out_rows * p.out_cols)


def resnet50_v15(batch):
    """ResNet-50 v1.5 conv stack: 7x7/2 stem (explicit pad 3, the reference's 230x230 VALID entry,
    bench/conv2d/resnet_params.def:122), 3x3/2 SAME max pool, bottleneck stages [3,4,6,3] with mid
    widths 64/128/256/512 and expansion 4, stride 2 on the 3x3 of the first block of stages 2-4,
    1x1 projection shortcuts on first blocks, global 7x7 average pool.  Buffers are named; a
    layer reads ``src`` and writes ``dst``."""
    layers = []
    layers.append(ConvLayer("stem", api.conv_params(batch, 224, 224, 3, 64, 7, 2, pad=3), "input", "a"))
    layers.append(PoolLayer("stem_pool", api.POOL_MAX, api.pool_params(batch, 112, 112, 64, 3, 2, True), "a", "b"))
    size, cin, cur = 56, 64, "b"
    names = ["a", "b", "c", "d", "e"]
    for stage, (blocks, mid) in enumerate(zip((3, 4, 6, 3), (64, 128, 256, 512)), start=1):
        cout = mid * 4
        for blk in range(blocks):
            stride = 2 if (blk == 0 and stage > 1) else 1
            free = [n for n in names if n != cur]
            t1, t2, t3, t4 = free[0], free[1], free[2], free[3]
            tag = "s%db%d" % (stage, blk + 1)
            if blk == 0:
                layers.append(ConvLayer(tag + "_proj", api.conv_params(batch, size, size, cin, cout, 1, stride), cur, t4))
            layers.append(ConvLayer(tag + "_1x1a", api.conv_params(batch, size, size, cin, mid, 1, 1), cur, t1))
            layers.append(ConvLayer(tag + "_3x3", api.conv_params(batch, size, size, mid, mid, 3, stride), t1, t2))
            size_out = size // stride
            layers.append(ConvLayer(tag + "_1x1b", api.conv_params(batch, size_out, size_out, mid, cout, 1, 1), t2, t3))
            cur, cin, size = t3, cout, size_out
    layers.append(PoolLayer("global_pool", api.POOL_AVERAGE, api.pool_params(batch, 7, 7, 2048, 7, 1, False), cur, "out"))
    return layers


def vgg16(batch):
    """VGG-16 conv stack: thirteen 3x3/1 SAME layers, 2x2/2 VALID max pool after each stage
    (shapes as bench/conv2d/vgg_params.def:46-54)."""
    layers, size, cin, cur, other = [], 224, 3, "input", "a"
    for stage, (reps, width) in enumerate(((2, 64), (2, 128), (3, 256), (3, 512), (3, 512)), start=1):
        for i in range(reps):
            dst = "a" if cur != "a" else "b"
            layers.append(ConvLayer("conv%d_%d" % (stage, i + 1), api.conv_params(batch, size, size, cin, width, 3, 1), cur, dst))
            cur, cin = dst, width
        dst = "a" if cur != "a" else "b"
        layers.append(PoolLayer("pool%d" % stage, api.POOL_MAX, api.pool_params(batch, size, size, cin, 2, 2, False), cur, dst))
        cur, size = dst, size // 2
    return layers


def mobilenet_v2_depthwise(batch):
    """The 17 depthwise 3x3 layers of MobileNet-v2 as (in_size, channels, stride)."""
    shapes = [(112, 32, 1), (112, 96, 2), (56, 144, 1), (56, 144, 2), (28, 192, 1), (28, 192, 1), (28, 192, 2),
              (14, 384, 1), (14, 384, 1), (14, 384, 1), (14, 384, 1), (14, 576, 1), (14, 576, 1), (14, 576, 2),
              (7, 960, 1), (7, 960, 1), (7, 960, 1)]
    return [api.depthwise_params(batch, s, s, c, 1, 3, st, True) for (s, c, st) in shapes]


def conv_flops(layers):
    return sum(l.flops for l in layers if isinstance(l, ConvLayer))
