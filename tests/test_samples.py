"""The two inference samples (samples/networks/vgg16.cc, resnet50.cc): they must compile as plain C++17
against the layer wrappers, and on a GPU their class probabilities must equal the same networks
recomputed layer by layer with the CPU oracle from the same seeded tensors (the hash of
samples/networks/sample_common.h restated in numpy)."""
import os
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")
SAMPLES = ["vgg16", "resnet50"]


def _build(name):
    from portdnn_b200 import build
    build.build()
    src_dir = os.path.join(ROOT, "samples", "networks")
    out_dir = os.path.join(ROOT, "samples", "networks", "_obj")
    os.makedirs(out_dir, exist_ok=True)
    exe = os.path.join(out_dir, name)
    deps = [os.path.join(src_dir, name + ".cc"), os.path.join(src_dir, "sample_common.h"),
            os.path.join(ROOT, "include", "portdnn_b200.h")]
    for sub in ("portdnn", "tools"):
        for d, _, files in os.walk(os.path.join(ROOT, "include", sub)):
            deps += [os.path.join(d, f) for f in files]
    if os.path.exists(exe) and all(os.path.getmtime(exe) >= os.path.getmtime(d) for d in deps):
        return exe
    cmd = ["g++", "-std=c++17", "-O2", "-Wall", "-I" + os.path.join(ROOT, "include"), "-I" + src_dir,
           "-I" + os.path.join(CUDA, "include"), os.path.join(src_dir, name + ".cc"),
           "-L" + os.path.join(ROOT, "portdnn_b200"), "-lportdnn_b200", "-L" + os.path.join(CUDA, "lib64"), "-lcudart",
           "-Wl,-rpath," + os.path.join(ROOT, "portdnn_b200"), "-Wl,-rpath," + os.path.join(CUDA, "lib64"), "-o", exe]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    assert res.returncode == 0, res.stdout
    return exe


@pytest.mark.parametrize("name", SAMPLES)
def test_samples_compile_and_link(name):
    assert os.path.exists(_build(name))


def hashed_tensor(n, seed, scale, offset=0.0):
    """sample::hashed_tensor: offset + scale * (murmur3 finaliser of the index and the seed, mapped to [-1, 1))."""
    with np.errstate(over="ignore"):
        x = (np.arange(n, dtype=np.uint32) * np.uint32(2654435761)) ^ np.uint32((seed * 0x9E3779B9) & 0xFFFFFFFF)
        x ^= x >> np.uint32(16)
        x *= np.uint32(0x85EBCA6B)
        x ^= x >> np.uint32(13)
        x *= np.uint32(0xC2B2AE35)
        x ^= x >> np.uint32(16)
    unit = (x >> np.uint32(8)).astype(np.float32) * np.float32(2.0 / 16777216.0) - np.float32(1.0)
    return (np.float32(offset) + np.float32(scale) * unit).astype(np.float32)


class OracleChain:
    """The layers of sample::Chain on the CPU; seeds count up in the same order."""

    def __init__(self, orc, batch, gain=2.0):
        self.orc, self.batch, self.seed, self.gain = orc, batch, 1, np.float32(gain)
        self.x = hashed_tensor(batch * 224 * 224 * 3, 0, 1.0)
        self.size, self.channels = 224, 3

    def _next(self):
        self.seed += 1
        return self.seed - 1

    def conv(self, features, window, stride, same):
        p = self.orc.conv_params(self.batch, self.size, self.size, self.channels, features, window, stride, same)
        fan_in = window * window * self.channels
        w = hashed_tensor(fan_in * features, self._next(), np.sqrt(np.float32(3.0) * self.gain / np.float32(fan_in)))
        self.x = self.orc.conv2d(self.orc.FORWARD, self.x, w, p)
        self.size, self.channels = p.out_rows, features

    def bias(self):
        b = hashed_tensor(self.channels, self._next(), 0.1)
        self.x = (self.x.reshape(-1, self.channels) + b).astype(np.float32).ravel()

    def relu(self):
        self.x = np.maximum(self.x, 0)

    def batchnorm(self, eps):
        c = self.channels
        beta, gamma = hashed_tensor(c, self._next(), 0.1), hashed_tensor(c, self._next(), 0.5, 1.0)
        mean, var = hashed_tensor(c, self._next(), 0.1), hashed_tensor(c, self._next(), 0.5, 1.0)
        x = self.x.reshape(-1, c).astype(np.float64)
        self.x = ((x - mean) / np.sqrt(var.astype(np.float64) + eps) * gamma + beta).astype(np.float32).ravel()

    def pool(self, op, window, stride, same):
        p = self.orc.pool_params(self.batch, self.size, self.size, self.channels, window, stride, same)
        self.x = self.orc.pool_forward(op, self.x, p)
        self.size = p.out_rows

    def fc(self, out_features):
        width = self.x.size // self.batch
        w = hashed_tensor(width * out_features, self._next(), np.sqrt(np.float32(3.0) * self.gain / np.float32(width)))
        self.x = (self.x.reshape(self.batch, width).astype(np.float64) @ w.reshape(width, out_features).astype(np.float64)
                  ).astype(np.float32).ravel()
        self.size, self.channels = 1, out_features

    def softmax(self):
        x = self.x.reshape(self.batch, -1).astype(np.float64)
        e = np.exp(x - x.max(axis=1, keepdims=True))
        return (e / e.sum(axis=1, keepdims=True)).astype(np.float32).ravel()


def vgg16_reference(orc, batch):
    net = OracleChain(orc, batch)
    for layers, features in ((2, 64), (2, 128), (3, 256), (3, 512), (3, 512)):
        for _ in range(layers):
            net.conv(features, 3, 1, True)
            net.bias()
            net.relu()
        net.pool(orc.POOL_MAX, 2, 2, False)
    for i, features in enumerate((4096, 4096, 1000)):
        net.fc(features)
        net.bias()
        if i < 2:
            net.relu()
    return net.softmax()


def resnet50_reference(orc, batch):
    net, eps = OracleChain(orc, batch, gain=1.0), 1.001e-5

    def unit(features, window, stride, same, relu):
        net.conv(features, window, stride, same)
        net.bias()
        net.batchnorm(eps)
        if relu:
            net.relu()

    unit(64, 7, 2, True, True)
    net.pool(orc.POOL_MAX, 3, 2, True)
    for stage, (blocks, mid) in enumerate(((3, 64), (4, 128), (6, 256), (3, 512))):
        for block in range(blocks):
            stride = 2 if (block == 0 and stage > 0) else 1
            state = (net.x, net.size, net.channels)
            shortcut = net.x
            if block == 0:
                unit(4 * mid, 1, stride, False, False)
                shortcut = net.x
                net.x, net.size, net.channels = state
            unit(mid, 1, stride, True, True)
            unit(mid, 3, 1, True, True)
            unit(4 * mid, 1, 1, True, False)
            net.x = (net.x + shortcut).astype(np.float32)
            net.relu()
    net.pool(orc.POOL_AVERAGE, net.size, 1, False)
    net.fc(1000)
    net.bias()
    return net.softmax()


@pytest.mark.gpu
@pytest.mark.parametrize("name", SAMPLES)
def test_sample_matches_oracle_network(orc, name, tmp_path):
    exe = _build(name)
    dump = str(tmp_path / (name + ".bin"))
    res = subprocess.run([exe, "--batch", "1", "--iterations", "2", "--dump", dump], stdout=subprocess.PIPE,
                         stderr=subprocess.STDOUT, text=True, timeout=600)
    assert res.returncode == 0, res.stdout
    assert "classed as" in res.stdout and res.stdout.count(" ns") == 2, res.stdout
    got = np.fromfile(dump, dtype=np.float32)
    ref = (vgg16_reference if name == "vgg16" else resnet50_reference)(orc, 1)
    assert got.size == ref.size == 1000
    assert abs(float(got.sum()) - 1.0) < 1e-4
    assert int(got.argmax()) == int(ref.argmax())
    # fp32 tensors through the 3xTF32 convolutions (1e-4 per layer) and the fp32 softmax
    assert np.abs(got - ref).max() <= 2e-3 * ref.max(), (float(np.abs(got - ref).max()), float(ref.max()))
