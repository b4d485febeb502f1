"""ResNet-152 on CIFAR-10-shaped inputs: images / s of a full training step (forward, loss, backward, AdamW).

``python -m cverl_b200.cli.resnet_cifar10_bench [--data-dir data/cifar10] [--steps 20] [--warmup 5] [--batch-size 128]
[--dtype bfloat16] [--channels-last] [--depth 152]``

With ``--data-dir`` it maps the tensors written by ``cverl_b200.cli.export_cifar10_tensors`` (``train_images.f32``,
``train_labels.i64``, ``train_meta.json``); otherwise it draws normal inputs of the same shape.  Timing is CUDA
events around the timed steps after the warm-up (wall clock on CPU), every step copies its batch from pinned host
memory.  The optimizer is this package's ``Fp32MasterAdamW``.  The network is the standard bottleneck ResNet
(3-8-36-3 blocks for depth 152) with a 3 x 3 stem for 32 x 32 inputs; it is convolution work for the vendor library
and serves as a non-language-model baseline of the framework layer, like the reference's C++ / Python pair
(tools/bench/resnet152_cifar10_cpp_bench.cc, resnet152_cifar10_python_bench.py).
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from pathlib import Path

import numpy as np
import torch
import torch.nn.functional as F

from ..optim import AdamWOptions, Fp32MasterAdamW

BLOCKS = {50: (3, 4, 6, 3), 101: (3, 4, 23, 3), 152: (3, 8, 36, 3), 14: (1, 1, 1, 1)}


class Bottleneck(torch.nn.Module):
    def __init__(self, cin: int, mid: int, stride: int):
        super().__init__()
        cout = mid * 4
        self.c1 = torch.nn.Conv2d(cin, mid, 1, bias=False)
        self.b1 = torch.nn.BatchNorm2d(mid)
        self.c2 = torch.nn.Conv2d(mid, mid, 3, stride=stride, padding=1, bias=False)
        self.b2 = torch.nn.BatchNorm2d(mid)
        self.c3 = torch.nn.Conv2d(mid, cout, 1, bias=False)
        self.b3 = torch.nn.BatchNorm2d(cout)
        self.down = None
        if stride != 1 or cin != cout:
            self.down = torch.nn.Sequential(torch.nn.Conv2d(cin, cout, 1, stride=stride, bias=False),
                                            torch.nn.BatchNorm2d(cout))

    def forward(self, x):
        y = F.relu(self.b1(self.c1(x)))
        y = F.relu(self.b2(self.c2(y)))
        y = self.b3(self.c3(y))
        return F.relu(y + (x if self.down is None else self.down(x)))


class ResNet(torch.nn.Module):
    def __init__(self, depth: int = 152, classes: int = 10, width: int = 64):
        super().__init__()
        self.stem = torch.nn.Sequential(torch.nn.Conv2d(3, width, 3, padding=1, bias=False), torch.nn.BatchNorm2d(width),
                                        torch.nn.ReLU())
        layers, cin = [], width
        for stage, n in enumerate(BLOCKS[depth]):
            mid = width * 2 ** stage
            for b in range(n):
                layers.append(Bottleneck(cin, mid, 2 if (b == 0 and stage > 0) else 1))
                cin = mid * 4
        self.layers = torch.nn.Sequential(*layers)
        self.fc = torch.nn.Linear(cin, classes)

    def forward(self, x):
        x = self.layers(self.stem(x))
        return self.fc(F.adaptive_avg_pool2d(x, 1).flatten(1))


def load_tensors(data_dir: Path, split: str = "train"):
    meta = json.loads((data_dir / f"{split}_meta.json").read_text())
    shape = tuple(meta["shape"])
    x = np.memmap(data_dir / f"{split}_images.f32", dtype=np.float32, mode="r", shape=shape)
    y = np.memmap(data_dir / f"{split}_labels.i64", dtype=np.int64, mode="r", shape=(shape[0],))
    return torch.from_numpy(np.ascontiguousarray(x)), torch.from_numpy(np.ascontiguousarray(y))


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--data-dir", default="")
    ap.add_argument("--device", default="cuda:0" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch-size", type=int, default=128)
    ap.add_argument("--dtype", default="bfloat16", choices=["float32", "bfloat16"])
    ap.add_argument("--channels-last", action="store_true")
    ap.add_argument("--depth", type=int, default=152, choices=sorted(BLOCKS))
    ap.add_argument("--width", type=int, default=64)
    ap.add_argument("--lr", type=float, default=1e-3)
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    torch.manual_seed(a.seed)
    device = torch.device(a.device)
    cuda = device.type == "cuda"
    if a.data_dir:
        x, y = load_tensors(Path(a.data_dir))
    else:
        n = max(a.batch_size * 4, 512)
        x, y = torch.randn(n, 3, 32, 32), torch.randint(0, 10, (n,))
    if cuda:
        x, y = x.pin_memory(), y.pin_memory()
    model = ResNet(a.depth, 10, a.width).to(device)
    if a.channels_last:
        model = model.to(memory_format=torch.channels_last)
    params = list(model.parameters())
    opt = Fp32MasterAdamW(params, AdamWOptions(lr=a.lr, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01,
                                               use_master_weights=False))
    amp = torch.bfloat16 if a.dtype == "bfloat16" else None
    n = x.shape[0]

    def step(i: int):
        lo = (i * a.batch_size) % max(n - a.batch_size + 1, 1)
        xb = x[lo:lo + a.batch_size].to(device, non_blocking=True)
        yb = y[lo:lo + a.batch_size].to(device, non_blocking=True)
        if a.channels_last:
            xb = xb.contiguous(memory_format=torch.channels_last)
        for p in params:
            p.grad = None
        with torch.autocast(device.type, dtype=amp, enabled=amp is not None):
            loss = F.cross_entropy(model(xb).float(), yb)
        loss.backward()
        opt.step()
        return loss.detach()

    first = None
    for i in range(a.warmup):
        first = step(i) if first is None else first
        step(i)
    if cuda:
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    t0 = time.perf_counter()
    for i in range(a.steps):
        last = step(a.warmup + i)
    if cuda:
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
    else:
        ms = (time.perf_counter() - t0) * 1e3
    out = {"benchmark": f"resnet{a.depth}_cifar10_train_step", "device": str(device), "dtype": a.dtype,
           "channels_last": a.channels_last, "batch_size": a.batch_size, "steps": a.steps, "warmup": a.warmup,
           "ms_per_step": ms / a.steps, "images_per_s": a.batch_size * a.steps / (ms / 1e3),
           "parameters": sum(p.numel() for p in params), "loss": float(last),
           "data": a.data_dir or "synthetic normal inputs", "timer": "CUDA events" if cuda else "wall clock"}
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
