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
    1x1 projection shortcuts on first blocks (bias only: the shortcut branch of the network has no
    ReLU of its own), global 7x7 average pool.  Buffers are named; a
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
                layers.append(ConvLayer(tag + "_proj", api.conv_params(batch, size, size, cin, cout, 1, stride), cur, t4,
                                        api.ACT_NONE))
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


def mobilenet_v2_convs(batch):
    """The dense convolutions of MobileNet-v2 at 224x224: the 3x3/2 stem and, per inverted-residual block,
    the 1x1 expansion (ReLU6; absent when the expansion factor is 1) and the linear 1x1 projection.
    Schedule (t, c, n, s) = (1,16,1,1)(6,24,2,2)(6,32,3,2)(6,64,4,2)(6,96,3,1)(6,160,3,2)(6,320,1,1).  The
    depthwise layers between them are mobilenet_v2_depthwise(); each layer here reads one buffer and
    writes the other, which is all a timing run needs."""
    layers = [ConvLayer("stem", api.conv_params(batch, 224, 224, 3, 32, 3, 2), "input", "a", api.ACT_RELU6)]
    size, cin, k = 112, 32, 0
    for t, c, n, s in ((1, 16, 1, 1), (6, 24, 2, 2), (6, 32, 3, 2), (6, 64, 4, 2), (6, 96, 3, 1), (6, 160, 3, 2), (6, 320, 1, 1)):
        for i in range(n):
            stride = s if i == 0 else 1
            k += 1
            hidden = cin * t
            if t != 1:
                layers.append(ConvLayer("b%d_expand" % k, api.conv_params(batch, size, size, cin, hidden, 1, 1), "a", "b", api.ACT_RELU6))
            size //= stride  # the depthwise layer in between changes the resolution
            layers.append(ConvLayer("b%d_project" % k, api.conv_params(batch, size, size, hidden, c, 1, 1), "b", "a", api.ACT_NONE))
            cin = c
    return layers


def conv_flops(layers):
    return sum(l.flops for l in layers if isinstance(l, ConvLayer))


class ConvStackRunner:
    """Runs a layer table on one GPU through the C ABI: forward only (activations ping-pong
    between a few named buffers) or a training step (every activation kept; then, last layer
    first, ReLU gradient -> filter backprop -> input backprop per convolution, max-pool gradient
    for pooling layers, filter gradients written as fp32 into one contiguous bucket and summed
    over ranks, stage by stage or with a single all-reduce).  The reference has no trainer; its samples chain layers the
    same way on the host (tools/network.h)."""

    def __init__(self, layers, device, seed, training=False, dtype=None, chunk=None, chunk_layers=0,
                 fuse_accumulate=True, bitmasks=True):
        """bitmasks (training, 16-bit): every convolution with a ReLU also writes the sign bits of its output (one
        bit per element), and the input backprops read those instead of the output tensor for the ReLU mask.
        fuse_accumulate (training): a gradient with several contributions is summed (and masked) inside the
        input backprops that bring them (PdnnBackpropFusion.accumulate); False keeps the unfused chain of an
        input backprop into a temporary, an add and a ReLU-gradient pass.
        chunk / chunk_layers (forward only): the first ``chunk_layers`` layers run depth-first over
        slices of ``chunk`` images - all those layers on images 0..chunk-1, then on the next slice, and so
        on - with their intermediate activations in slice-sized buffers that every slice reuses, so that a
        layer's output is still in the L2 cache when the next layer reads it.  Results are identical to
        the layer-by-layer order: every operator of the path is independent per image."""
        import torch
        from . import dist as pdist
        self.torch, self.layers, self.training, self.device = torch, layers, training, device
        self.fuse_accumulate = fuse_accumulate
        self.use_bits = bool(bitmasks and training and self.dtype_is_16bit(dtype, torch))
        self.dtype = dtype or torch.float16
        self.code = api.F16 if self.dtype == torch.float16 else api.BF16 if self.dtype == torch.bfloat16 else api.F32
        g = torch.Generator(device=device).manual_seed(seed)
        self.weights, self.biases, self.workspaces = {}, {}, {}
        first = layers[0].params
        self.input = torch.randn(first.batch * first.in_rows * first.in_cols * first.channels, device=device,
                                 generator=g).to(self.dtype)
        # dataflow: which tensor (index of the producing layer, -1 = network input) each layer reads
        current, self.src_idx, sizes = {layers[0].src: -1}, [], []
        for i, l in enumerate(layers):
            p = l.params
            self.src_idx.append(current.get(l.src, -2))  # -2: a buffer nobody has written (timing-only tables)
            current[l.dst] = i
            if isinstance(l, ConvLayer):
                fan_in = p.window_rows * p.window_cols * p.channels
                w = torch.randn(fan_in * p.features, device=device, generator=g) * (2.0 / fan_in) ** 0.5  # He-normal
                self.weights[i] = w.to(self.dtype)
                self.biases[i] = (torch.randn(p.features, device=device, generator=g) * 0.01).to(self.dtype)
                sizes.append(p.batch * p.out_rows * p.out_cols * p.features)
                _, rec = api.conv2d_workspace_size(api.FORWARD, self.code, p, api.ALGO_IM2COL)
                if rec:
                    self.workspaces[i] = torch.empty(rec, dtype=self.dtype, device=device)
            else:
                sizes.append(p.batch * p.out_rows * p.out_cols * p.channels)
        self.sizes = sizes
        self.flops_forward = conv_flops(layers)
        if training:
            self.acts = [torch.empty(n, dtype=self.dtype, device=device) for n in sizes]
            # sign bits of the ReLU outputs (a sixteenth of the tensors' bytes), where the layer shape allows
            self.bits = {i: torch.empty(sizes[i] // 8, dtype=torch.uint8, device=device)
                         for i, l in enumerate(layers)
                         if self.use_bits and isinstance(l, ConvLayer) and l.activation == api.ACT_RELU and
                         l.params.features % 8 == 0 and self._bitmask_pays(l)}
            self.grads = [None] * len(layers)
            conv_ids = [i for i, l in enumerate(layers) if isinstance(l, ConvLayer)]
            self.conv_ids = conv_ids
            self.bucket = pdist.FilterGradientBucket([self.weights[i].numel() for i in conv_ids], device,
                                                     pad_to=25_500_000)
            self.scratch = torch.empty(max(sizes), dtype=self.dtype, device=device)
            last = conv_ids[-1]
            self.dy_last = torch.randn(sizes[last], device=device, generator=g).to(self.dtype)
            self.fbp_ws = {}
            for i in conv_ids:
                _, rec = api.conv2d_workspace_size(api.FILTER_BACKPROP, self.code, layers[i].params, api.ALGO_IM2COL)
                if rec:
                    self.fbp_ws[i] = rec
            self.fbp_workspace = torch.empty(max(self.fbp_ws.values(), default=1), dtype=self.dtype, device=device)
            # forward + filter backprop everywhere, input backprop everywhere but the first layer
            self.flops_train = sum(l.flops * (3 if self.src_idx[i] != -1 else 2)
                                   for i, l in enumerate(layers) if isinstance(l, ConvLayer))
        else:
            names = {}
            for l, n in zip(layers, sizes):
                names[l.dst] = max(names.get(l.dst, 0), n)
            self.buffers = {k: torch.empty(v, dtype=self.dtype, device=device) for k, v in names.items()}
        self.chunk, self.chunk_layers = None, 0
        if chunk and chunk_layers and not training and first.batch % chunk == 0 and chunk < first.batch:
            self.chunk, self.chunk_layers, batch = chunk, chunk_layers, first.batch
            # only the last layer of the depth-first part may be read by a later layer
            assert all(j == chunk_layers - 1 or j >= chunk_layers for j in self.src_idx[chunk_layers:])
            self.chunk_params, names = [], {}
            for i in range(chunk_layers):
                q = type(layers[i].params).from_buffer_copy(layers[i].params)
                q.batch = chunk
                self.chunk_params.append(q)
                names[layers[i].dst] = max(names.get(layers[i].dst, 0), sizes[i] // batch * chunk)
            self.chunk_buffers = {k: torch.empty(v, dtype=self.dtype, device=device) for k, v in names.items()}

    @staticmethod
    def _bitmask_pays(l):
        """Reading the sign bits instead of the output tensor saves an input backprop 5-22 us; writing them costs
        the forward layer 0.5-4 us.  Measured over the whole step, bits for the outputs of the 1x1 expansions
        as well change nothing (forward +0.06 ms, backward -0.06 ms), so those keep the tensor form.  The
        stem's output is masked inside the pool gradient and needs none."""
        p = l.params
        expansion = p.window_rows == 1 and p.features >= 4 * p.channels
        return not expansion and l.src != "input"

    @staticmethod
    def dtype_is_16bit(dtype, torch):
        return dtype is None or dtype in (torch.float16, torch.bfloat16)

    # ---- forward -------------------------------------------------------------------------------
    def _out(self, i):
        return self.acts[i] if self.training else self.buffers[self.layers[i].dst][:self.sizes[i]]

    def _in(self, i):
        j = self.src_idx[i]
        p = self.layers[i].params
        n_in = p.batch * p.in_rows * p.in_cols * p.channels
        if j == -2:  # read the named buffer as it is
            return self.buffers[self.layers[i].src][:n_in]
        t = self.input if j < 0 else self._out(j)
        # timing-only tables leave out layers in between (a strided depthwise layer): read what fits
        return t if t.numel() == n_in else t[:n_in]

    def run_layer(self, i):
        l, p = self.layers[i], self.layers[i].params
        if isinstance(l, ConvLayer):
            api.conv2d(api.FORWARD, self._in(i), self.weights[i], p, algorithm=api.ALGO_IM2COL, out=self._out(i),
                       bias=self.biases[i], activation=l.activation, workspace=self.workspaces.get(i),
                       relu_bitmask=self.bits.get(i) if self.training else None,
                       constant_filter=True)  # the weights are not written inside a step
        else:
            api.pooling(l.op, 0, self._in(i), p, out=self._out(i))

    def run_layer_slice(self, i, c):
        """Layer i (one of the depth-first layers) on images [c * chunk, (c + 1) * chunk)."""
        l, p, j = self.layers[i], self.chunk_params[i], self.src_idx[i]
        batch = self.layers[0].params.batch
        n_out = self.sizes[i] // batch * self.chunk
        if j < 0:
            n_in = self.input.numel() // batch * self.chunk
            src = self.input[c * n_in:(c + 1) * n_in]
        else:
            src = self.chunk_buffers[self.layers[j].dst][:self.sizes[j] // batch * self.chunk]
        if i == self.chunk_layers - 1:  # the part's result goes to its place in the full-batch tensor
            dst = self._out(i)[c * n_out:(c + 1) * n_out]
        else:
            dst = self.chunk_buffers[l.dst][:n_out]
        if isinstance(l, ConvLayer):
            api.conv2d(api.FORWARD, src, self.weights[i], p, algorithm=api.ALGO_IM2COL, out=dst, bias=self.biases[i],
                       activation=l.activation, workspace=self.workspaces.get(i))
        else:
            api.pooling(l.op, 0, src, p, out=dst)

    def forward(self):
        first = 0
        if self.chunk:
            first = self.chunk_layers
            for c in range(self.layers[0].params.batch // self.chunk):
                for i in range(first):
                    self.run_layer_slice(i, c)
        for i in range(first, len(self.layers)):
            self.run_layer(i)
        return self._out(len(self.layers) - 1)

    # ---- backward ------------------------------------------------------------------------------
    def _plan_backward(self):
        """Which tensors get their ReLU-gradient mask applied inside the input backprop that completes
        their gradient (a convolution's output whose unmasked gradient nobody else needs; with several
        readers the last one to arrive adds to the others' sum and masks it), and the segments of the
        backward pass: the layers of one stage, last stage first, each with the slice of the gradient
        bucket it fills."""
        layers = self.layers
        readers = [0] * len(layers)
        for j in self.src_idx:
            if j >= 0:
                readers[j] += 1
        self.readers = readers
        self.fuse_mask = [isinstance(l, ConvLayer) and l.activation == api.ACT_RELU and
                          (readers[i] == 1 or (readers[i] > 1 and self.fuse_accumulate))
                          for i, l in enumerate(layers)]
        stage_of = lambda l: l.name[:2] if l.name[0] == "s" and l.name[1].isdigit() else "stem"
        self.segments = []
        for i in reversed(range(len(layers))):
            tag = stage_of(layers[i])
            if not self.segments or self.segments[-1]["tag"] != tag:
                self.segments.append({"tag": tag, "layers": []})
            self.segments[-1]["layers"].append(i)
        for seg in self.segments:
            ks = [self.conv_ids.index(i) for i in seg["layers"] if i in self.weights]
            seg["bucket"] = self.bucket.span(min(ks), max(ks)) if ks else None

    def _add_grad(self, j, producer):
        """Routes a gradient into tensor j: the first contribution is written in place, later ones
        are accumulated.  producer(dst, accumulate) writes (or adds) its gradient into dst, or returns
        False if it cannot add in place, in which case it is asked again for a temporary."""
        if self.grads[j] is None:
            self.grads[j] = self.torch.empty(self.sizes[j], dtype=self.dtype, device=self.device)
        if j not in self._fresh:
            producer(self.grads[j], False)
            self._fresh.add(j)
        elif producer(self.grads[j], True) is False:
            tmp = self.scratch2[:self.sizes[j]]
            producer(tmp, False)
            api.scale_blend(tmp, 1.0, self.grads[j], 1.0, out=self.grads[j])

    def backward_begin(self):
        if not hasattr(self, "segments"):
            self._plan_backward()
            self.scratch2 = self.torch.empty_like(self.scratch)
        self._fresh, self._masked, self._block_grad = set(), set(), {}

    def backward_segment(self, seg):
        """The backward pass of one segment: per convolution (last first) the ReLU gradient - unless the
        input backprop that produced the incoming gradient already applied it - then the filter backprop,
        written as fp32 straight into the layer's slice of the gradient bucket, then the input backprop."""
        last = self.conv_ids[-1]
        if self.fuse_accumulate and seg["bucket"] is not None and self.dtype != self.torch.float32:
            # the filter backprops of this segment add their pixel splits straight into the bucket
            self.bucket.buffer[seg["bucket"][0]:seg["bucket"][1]].zero_()
        for i in seg["layers"]:
            l, p, j = self.layers[i], self.layers[i].params, self.src_idx[i]
            if i == last:
                dy = self.dy_last
            elif i in self._fresh:
                dy = self.grads[i]
            elif isinstance(l, ConvLayer) and l.name.endswith("_proj"):
                dy = self._block_grad[l.name[:-5]]  # the shortcut receives its block's output gradient
            else:
                continue  # nothing downstream of this layer takes part in the step (the final pool)
            if isinstance(l, ConvLayer):
                if i in self._masked or l.activation == api.ACT_NONE:
                    g = dy
                else:
                    g = self.scratch[:self.sizes[i]]
                    api.pointwise_grad(api.ACT_RELU, self.acts[i], dy, out=g)
                if l.name.endswith("_1x1b"):
                    # the block's output gradient after its ReLU: what the shortcut branch receives too
                    self._block_grad[l.name[:-5]] = g
                k = self.conv_ids.index(i)
                f32_out = self.dtype != self.torch.float32
                add = self.fuse_accumulate and f32_out
                api.conv2d(api.FILTER_BACKPROP, self._in(i), g, p, algorithm=api.ALGO_IM2COL, out=self.bucket.view(k),
                           output_f32=f32_out, accumulate=add,
                           workspace=self.fbp_workspace if i in self.fbp_ws else None)
                if j >= 0:
                    # The ReLU mask of tensor j goes into every input backprop that contributes to its
                    # gradient (the mask of a sum is the sum of the masked terms), so a later contribution
                    # adds to a gradient that is masked already and may skip what it does not reach.
                    mask = self.acts[j] if self.fuse_mask[j] else None

                    bits = self.bits.get(j) if mask is not None else None

                    def ibp(dst, accumulate, g=g, i=i, p=p, mask=mask, bits=bits):
                        if accumulate and not self.fuse_accumulate:
                            return False
                        masked = mask is not None and (accumulate or dst is self.grads[j])
                        api.conv2d(api.INPUT_BACKPROP, g, self.weights[i], p, algorithm=api.ALGO_IM2COL, out=dst,
                                   relu_forward_output=mask if (masked and bits is None) else None,
                                   relu_bitmask=bits if masked else None,
                                   accumulate=(2 if mask is not None else 1) if accumulate else 0, constant_filter=True)

                    self._add_grad(j, ibp)
                    if mask is not None:
                        self._masked.add(j)
            elif l.op == api.POOL_AVERAGE:
                if j >= 0:
                    self._add_grad(j, lambda dst, acc: False if acc else api.pooling(l.op, 1, dy, p, out=dst))
            elif j >= 0:
                # a pooled ReLU output with no other reader: its ReLU gradient rides on the pool gradient
                relu = (isinstance(self.layers[j], ConvLayer) and self.layers[j].activation == api.ACT_RELU and
                        self.readers[j] == 1 and self.fuse_accumulate)
                self._add_grad(j, lambda dst, acc: False if acc else
                               api.pooling_max_grad(l.op, self._in(i), self.acts[i], dy, p, out=dst, relu_input=relu))
                if relu:
                    self._masked.add(j)

    def backward(self):
        self.backward_begin()
        for seg in self.segments:
            self.backward_segment(seg)

    def train_step(self):
        self.forward()
        self.backward()
        return self.bucket.all_reduce()
