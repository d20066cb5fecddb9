"""Parity of the measured workloads as a whole: the layer tables of portdnn_b200/workloads.py run
through ConvStackRunner (the code bench.py times) against the CPU oracle chained layer by layer.

The reference chains layers on the host the same way (tools/network.h:26-79); every layer's
arithmetic is the direct kernel's (src/conv2d/direct/kernels_nhwc.h:62-130,206-278,356-420),
bias via binaryop Add, ReLU via pointwise (src/pointwise/kernels.h:181-237), pools via
src/pooling/kernels.h.  Each layer is checked on the GPU's OWN previous activation (so that
rounding does not compound), and the last tensor is also checked end to end against an oracle
chain that never sees a GPU value.

Parity bars: fp16 <= 2e-2, fp32 (3xTF32) <= 1e-4, in the sense of conftest.rel_err (max-norm and
element-wise); max pooling and the routing of its gradient bit-exact.  The end-to-end bars are
wider and stated where they are used.
"""
import numpy as np
import pytest
import torch

import portdnn_b200 as pd
from conftest import rel_err
from gpu_util import assert_no_device_error
from portdnn_b200 import workloads

pytestmark = pytest.mark.gpu


def host(t):
    return t.detach().float().cpu().numpy().ravel()


def half_round(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).half().float().numpy()


def oparams(orc, p):
    return orc.ConvParams(*[getattr(p, f) for f, _ in p._fields_])


def opool(orc, p):
    return orc.PoolParams(*[getattr(p, f) for f, _ in p._fields_])


def oracle_layer(orc, net, i, x, round_out):
    """Layer i of the runner's table on the host array x: conv + bias (+ ReLU), or the pool."""
    l, p = net.layers[i], net.layers[i].params
    if isinstance(l, workloads.ConvLayer):
        y = orc.conv2d(orc.FORWARD, x, host(net.weights[i]), oparams(orc, p))
        y = round_out(y)                                            # the convolution's own rounding
        y = round_out(y.reshape(-1, p.features) + host(net.biases[i])[None, :]).ravel()   # bias add
        return np.maximum(y, 0) if l.activation == pd.ACT_RELU else y   # ReLU
    return orc.pool_forward(l.op, x, opool(orc, p))


def check_forward(orc, net, tol, end_to_end_tol, round_out):
    net.forward()
    torch.cuda.synchronize()
    assert_no_device_error()
    chain = {-1: host(net.input)}
    worst, worst_name = 0.0, ""
    for i, l in enumerate(net.layers):
        j = net.src_idx[i]
        x_gpu = host(net.input if j < 0 else net.acts[j])
        got = host(net.acts[i])
        ref = oracle_layer(orc, net, i, x_gpu, round_out)
        if isinstance(l, workloads.PoolLayer) and l.op == pd.POOL_MAX:
            assert np.array_equal(got, ref), l.name
        else:
            e = rel_err(got, ref)
            if e > worst:
                worst, worst_name = e, l.name
            assert e <= tol, (l.name, e)
        chain[i] = oracle_layer(orc, net, i, chain[j], round_out)
    last = len(net.layers) - 1
    e2e = rel_err(host(net.acts[last]), chain[last])
    assert e2e <= end_to_end_tol, e2e
    return "%.2e (%s)" % (worst, worst_name), e2e


def test_resnet50_forward_every_layer_and_end_to_end(orc):
    net = workloads.ConvStackRunner(workloads.resnet50_v15(2), torch.device("cuda", 0), seed=11, training=True)
    # 55 chained layers: every fp16 rounding of an activation moves the next layer's input by up to
    # 2^-11 relative, so the end-to-end bar is 5e-2 while each single layer stays within 2e-2.
    worst, e2e = check_forward(orc, net, 2e-2, 5e-2, half_round)
    print("resnet50 b2 fp16: worst layer %s, end to end %.2e" % (worst, e2e))


def test_resnet50_depth_first_slices_equal_layer_by_layer():
    dev = torch.device("cuda", 0)
    a = workloads.ConvStackRunner(workloads.resnet50_v15(8), dev, seed=5)
    b = workloads.ConvStackRunner(workloads.resnet50_v15(8), dev, seed=5, chunk=2, chunk_layers=25)
    assert b.chunk == 2
    assert torch.equal(a.forward(), b.forward())
    assert_no_device_error()


def test_vgg16_fp32_forward_every_layer(orc):
    net = workloads.ConvStackRunner(workloads.vgg16(1), torch.device("cuda", 0), seed=3, training=True,
                                    dtype=torch.float32)
    worst, e2e = check_forward(orc, net, 1e-4, 1e-3, lambda a: a)
    print("vgg16 b1 fp32: worst layer %s, end to end %.2e" % (worst, e2e))


def test_mobilenet_v2_depthwise_layers(orc):
    rng = np.random.default_rng(17)
    for p in workloads.mobilenet_v2_depthwise(2):
        po = orc.DepthwiseParams(*[getattr(p, f) for f, _ in p._fields_])
        x = half_round(rng.standard_normal(p.batch * p.in_rows * p.in_cols * p.channels))
        f = half_round(rng.standard_normal(9 * p.channels) * 0.3)
        y = pd.depthwise_conv2d(pd.FORWARD, torch.from_numpy(x).cuda().half(), torch.from_numpy(f).cuda().half(), p)
        e = rel_err(host(y), orc.depthwise_conv2d(orc.FORWARD, x, f, po))
        assert e <= 2e-2, (p.in_rows, p.channels, p.stride_rows, e)


def test_mobilenet_v2_depthwise_layers_at_the_benchmark_batch(orc):
    """The 17 depthwise layers at the benchmark's batch of 128 (the launch heuristics - rows per thread,
    row segments, wave sizes - depend on the tensor sizes): forward of every layer, input and filter
    backprop of the four layers larger than L2 and of three small ones."""
    rng = np.random.default_rng(19)
    seen = set()
    for idx, p in enumerate(workloads.mobilenet_v2_depthwise(128)):
        key = (p.in_rows, p.channels, p.stride_rows)
        if key in seen:
            continue
        seen.add(key)
        po = orc.DepthwiseParams(*[getattr(p, f) for f, _ in p._fields_])
        x = half_round(rng.standard_normal(p.batch * p.in_rows * p.in_cols * p.channels, dtype=np.float32))
        f = half_round(rng.standard_normal(9 * p.channels, dtype=np.float32) * 0.3)
        xd, fd = torch.from_numpy(x).cuda().half(), torch.from_numpy(f).cuda().half()
        e = rel_err(host(pd.depthwise_conv2d(pd.FORWARD, xd, fd, p)), orc.depthwise_conv2d(orc.FORWARD, x, f, po))
        assert e <= 2e-2, ("forward", key, e)
        if idx < 4 or key in ((28, 192, 2), (14, 576, 1), (7, 960, 1)):
            dy = half_round(rng.standard_normal(p.batch * p.out_rows * p.out_cols * p.channels, dtype=np.float32))
            dyd = torch.from_numpy(dy).cuda().half()
            e = rel_err(host(pd.depthwise_conv2d(pd.INPUT_BACKPROP, dyd, fd, p)),
                        orc.depthwise_conv2d(orc.INPUT_BACKPROP, dy, f, po))
            assert e <= 2e-2, ("input backprop", key, e)
            # sums of up to 1.6 million products per filter element, rounded once to fp16
            e = rel_err(host(pd.depthwise_conv2d(pd.FILTER_BACKPROP, xd, dyd, p)),
                        orc.depthwise_conv2d(orc.FILTER_BACKPROP, x, dy, po))
            assert e <= 2e-2, ("filter backprop", key, e)
    assert_no_device_error()


def test_resnet50_train_step_gradients(orc):
    """One training step at batch 2: every filter gradient in the bucket and every activation
    gradient the runner keeps, against oracle ReLU-gradient / filter-backprop / input-backprop /
    max-pool-gradient applied to the GPU's own incoming gradient of that layer."""
    net = workloads.ConvStackRunner(workloads.resnet50_v15(2), torch.device("cuda", 0), seed=23, training=True)
    net.forward()
    net.backward()
    torch.cuda.synchronize()
    assert_no_device_error()
    layers, last = net.layers, net.conv_ids[-1]
    block_grad, expect, checked_dw, checked_dx = {}, {}, 0, 0
    for i in reversed(range(len(layers))):
        l, p, j = layers[i], layers[i].params, net.src_idx[i]
        if i == last:
            dy, masked = host(net.dy_last), False
        elif net.grads[i] is not None:
            dy, masked = host(net.grads[i]), i in net._masked
        elif l.name.endswith("_proj"):
            dy, masked = block_grad[l.name[:-5]], False
        else:
            continue
        if isinstance(l, workloads.ConvLayer):
            # ReLU gradient (src/pointwise/kernels.h:205-233), unless the producing input backprop applied it
            # or the layer has no ReLU (the projection shortcuts)
            g = dy if (masked or l.activation == pd.ACT_NONE) else orc.pointwise_grad(0, host(net.acts[i]), dy)
            if masked:  # a masked gradient is zero wherever the activation is: the mask really was applied
                assert not np.any(dy[host(net.acts[i]) <= 0] != 0), l.name
            if l.name.endswith("_1x1b"):
                block_grad[l.name[:-5]] = g  # the shortcut branch receives the block's gradient after its ReLU
            x = host(net.input if j < 0 else net.acts[j])
            dw_ref = orc.conv2d(orc.FILTER_BACKPROP, x, g, oparams(orc, p))
            e = rel_err(host(net.bucket.view(net.conv_ids.index(i))), dw_ref)
            assert e <= 2e-2, ("dW", l.name, e)
            checked_dw += 1
            if j >= 0:
                dx = orc.conv2d(orc.INPUT_BACKPROP, g, host(net.weights[i]), oparams(orc, p))
                if net.fuse_mask[j]:
                    dx = orc.pointwise_grad(0, host(net.acts[j]), dx)
                expect[j] = expect.get(j, 0) + dx
        elif l.op == pd.POOL_MAX and j >= 0:
            dx = orc.pool_max_grad(l.op, host(net.acts[j]), host(net.acts[i]), dy, opool(orc, p))
            if j in net._masked:  # the pooled tensor's ReLU gradient is part of the pool-gradient call
                dx = orc.pointwise_grad(0, host(net.acts[j]), dx)
            expect[j] = expect.get(j, 0) + dx
        # every gradient that has received all its contributions by now is compared once
        for t in [t for t in expect if all(net.src_idx[r] != t or r >= i for r in range(len(layers)))]:
            e = rel_err(host(net.grads[t]), expect.pop(t))
            assert e <= 2e-2, ("dx into", layers[t].name, e)
            checked_dx += 1
    # 52 input backprops and the stem pool write 53 gradients into 49 tensors (4 block inputs have two readers)
    assert checked_dw == 53 and checked_dx == 49 and not expect, (checked_dw, checked_dx, list(expect))
    # the stem pool's gradient routing is exact: one contribution, copied values
    assert net.grads[0] is not None


def test_resnet50_train_step_at_the_benchmark_batch(orc):
    """The training step at the benchmark's batch of 256: the activation gradients of two sampled images (the
    input backprop is independent per image) through every layer, and the filter gradients - sums over the
    whole batch - of five layers that take different kernels (the few-channel stem, a 3x3 with two taps per
    tile, a strided 3x3, a strided projection without ReLU, a 7x7-pixel 1x1 expansion), against the oracle
    applied to the GPU's own incoming gradient of that layer."""
    batch, images = 256, (0, 255)
    full_dw = {"stem", "s1b1_3x3", "s2b1_3x3", "s3b1_proj", "s4b3_1x1b"}
    net = workloads.ConvStackRunner(workloads.resnet50_v15(batch), torch.device("cuda", 0), seed=29, training=True)
    net.forward()
    net.backward()
    torch.cuda.synchronize()
    assert_no_device_error()
    layers, last = net.layers, net.conv_ids[-1]

    def image_of(t, img):
        per = t.numel() // batch
        return host(t[img * per:(img + 1) * per])

    def one_image(p):
        q = type(p)(*[getattr(p, f) for f, _ in p._fields_])
        q.batch = 1
        return q

    def incoming(i, take):
        """(gradient arriving at layer i, whether the producing call already applied the ReLU mask) or None."""
        if i == last:
            return take(net.dy_last), False
        if net.grads[i] is not None:
            return take(net.grads[i]), i in net._masked
        return None

    checked_dx = 0
    for img in images:
        take = lambda t: image_of(t, img)
        block_grad, expect = {}, {}
        for i in reversed(range(len(layers))):
            l, p, j = layers[i], layers[i].params, net.src_idx[i]
            arriving = incoming(i, take)
            if arriving is None and l.name.endswith("_proj"):
                arriving = (block_grad[l.name[:-5]], False)
            if arriving is None:
                continue
            dy, masked = arriving
            if isinstance(l, workloads.ConvLayer):
                g = dy if (masked or l.activation == pd.ACT_NONE) else orc.pointwise_grad(0, take(net.acts[i]), dy)
                if l.name.endswith("_1x1b"):
                    block_grad[l.name[:-5]] = g
                if j >= 0:
                    dx = orc.conv2d(orc.INPUT_BACKPROP, g, host(net.weights[i]), oparams(orc, one_image(p)))
                    if net.fuse_mask[j]:
                        dx = orc.pointwise_grad(0, take(net.acts[j]), dx)
                    expect[j] = expect.get(j, 0) + dx
            elif l.op == pd.POOL_MAX and j >= 0:
                dx = orc.pool_max_grad(l.op, take(net.acts[j]), take(net.acts[i]), dy, opool(orc, one_image(p)))
                if j in net._masked:
                    dx = orc.pointwise_grad(0, take(net.acts[j]), dx)
                expect[j] = expect.get(j, 0) + dx
            for t in [t for t in expect if all(net.src_idx[r] != t or r >= i for r in range(len(layers)))]:
                e = rel_err(take(net.grads[t]), expect.pop(t))
                assert e <= 2e-2, ("dx into", layers[t].name, "image", img, e)
                checked_dx += 1
        assert not expect
    assert checked_dx == 49 * len(images), checked_dx

    checked_dw = 0
    block_grad_full = {}
    for i in reversed(range(len(layers))):
        l, p, j = layers[i], layers[i].params, net.src_idx[i]
        if not isinstance(l, workloads.ConvLayer):
            continue
        wanted = l.name in full_dw or (l.name.endswith("_1x1b") and l.name[:-5] + "_proj" in full_dw)
        if not wanted:
            continue
        arriving = incoming(i, host)
        if arriving is None and l.name.endswith("_proj"):
            arriving = (block_grad_full[l.name[:-5]], False)
        dy, masked = arriving
        g = dy if (masked or l.activation == pd.ACT_NONE) else orc.pointwise_grad(0, host(net.acts[i]), dy)
        if l.name.endswith("_1x1b"):
            block_grad_full[l.name[:-5]] = g
        if l.name not in full_dw:
            continue
        x = host(net.input if j < 0 else net.acts[j])
        dw_ref = orc.conv2d(orc.FILTER_BACKPROP, x, g, oparams(orc, p))
        e = rel_err(host(net.bucket.view(net.conv_ids.index(i))), dw_ref)
        assert e <= 2e-2, ("dW", l.name, e)
        checked_dw += 1
    assert checked_dw == len(full_dw), checked_dw
