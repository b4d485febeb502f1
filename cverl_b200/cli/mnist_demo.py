"""Small supervised demo of the framework layer on MNIST: IDX files -> 2 conv + 2 linear layers -> AdamW.

``python -m cverl_b200.cli.mnist_demo --data-dir data/mnist/raw [--device cuda:0] [--epochs 1] [--batch-size 256]
[--max-train-batches N] [--max-test-batches N] [--lr 1e-3] [--stop-when-train-acc-gt-test] [--metrics-csv f.csv]``

Reads the four raw IDX files (``train-images-idx3-ubyte`` ...; big-endian headers, magic 2051 / 2049), or draws a
synthetic ten-class problem with ``--synthetic`` when no data is at hand.  The optimizer is this package's
``Fp32MasterAdamW`` (the per-tensor AdamW of the RL trainers), so the demo doubles as its smoke test on a model
that is not a language model.  One CSV row per training step and one per epoch, with the reference demo's
columns (tools/torch/mnist_gpu_demo.cc:226-232); the run fails when the loss does not fall.
"""
from __future__ import annotations

import argparse
import struct
import sys
from pathlib import Path

import torch
import torch.nn.functional as F

from ..optim import AdamWOptions, Fp32MasterAdamW

COLUMNS = "step,epoch,batch,train_loss,train_accuracy,train_eval_loss,train_eval_accuracy,test_loss,test_accuracy"


def read_idx_images(path: Path) -> torch.Tensor:
    raw = path.read_bytes()
    magic, count, rows, cols = struct.unpack(">iiii", raw[:16])
    if magic != 2051 or count <= 0 or (rows, cols) != (28, 28) or len(raw) != 16 + count * rows * cols:
        raise ValueError(f"not an MNIST image IDX file: {path}")
    return torch.frombuffer(bytearray(raw[16:]), dtype=torch.uint8).view(count, 1, rows, cols).float().div_(255.0)


def read_idx_labels(path: Path) -> torch.Tensor:
    raw = path.read_bytes()
    magic, count = struct.unpack(">ii", raw[:8])
    if magic != 2049 or count <= 0 or len(raw) != 8 + count:
        raise ValueError(f"not an MNIST label IDX file: {path}")
    return torch.frombuffer(bytearray(raw[8:]), dtype=torch.uint8).long()


def load_split(data_dir: Path, train: bool):
    stem = "train" if train else "t10k"
    x = read_idx_images(data_dir / f"{stem}-images-idx3-ubyte")
    y = read_idx_labels(data_dir / f"{stem}-labels-idx1-ubyte")
    if x.shape[0] != y.shape[0]:
        raise ValueError("image / label count mismatch")
    return x, y


def synthetic_split(n: int, seed: int):
    """Ten classes of 28 x 28 images: a class-specific blob pattern plus noise (separable, not trivial)."""
    g = torch.Generator().manual_seed(1234)
    protos = torch.rand(10, 1, 28, 28, generator=g)
    g2 = torch.Generator().manual_seed(seed)
    y = torch.randint(0, 10, (n,), generator=g2)
    x = (0.6 * protos[y] + 0.4 * torch.rand(n, 1, 28, 28, generator=g2)).clamp_(0, 1)
    return x, y


class Net(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.conv1 = torch.nn.Conv2d(1, 32, 3, padding=1)
        self.conv2 = torch.nn.Conv2d(32, 64, 3, padding=1)
        self.fc1 = torch.nn.Linear(64 * 7 * 7, 128)
        self.fc2 = torch.nn.Linear(128, 10)

    def forward(self, x):
        x = F.max_pool2d(F.relu(self.conv1(x)), 2)
        x = F.max_pool2d(F.relu(self.conv2(x)), 2)
        x = F.dropout(F.relu(self.fc1(x.flatten(1))), 0.25, self.training)
        return self.fc2(x)


@torch.no_grad()
def evaluate(model, x, y, device, batch_size: int, max_batches: int):
    model.eval()
    loss_sum, correct, seen = 0.0, 0, 0
    for b, lo in enumerate(range(0, x.shape[0], batch_size)):
        if max_batches > 0 and b >= max_batches:
            break
        xb, yb = x[lo:lo + batch_size].to(device), y[lo:lo + batch_size].to(device)
        logits = model(xb)
        loss_sum += float(F.cross_entropy(logits, yb)) * xb.shape[0]
        correct += int((logits.argmax(1) == yb).sum())
        seen += xb.shape[0]
    if seen == 0:
        raise RuntimeError("evaluation saw zero examples")
    return loss_sum / seen, correct / seen


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--data-dir", default="data/mnist/raw")
    ap.add_argument("--synthetic", action="store_true", help="draw a synthetic ten-class problem instead of reading IDX files")
    ap.add_argument("--device", default="cuda:0" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--metrics-csv", default="")
    ap.add_argument("--epochs", type=int, default=1)
    ap.add_argument("--batch-size", type=int, default=256)
    ap.add_argument("--max-train-batches", type=int, default=0, help="0 = the whole epoch")
    ap.add_argument("--max-test-batches", type=int, default=0, help="0 = the whole test split")
    ap.add_argument("--lr", type=float, default=1e-3)
    ap.add_argument("--seed", type=int, default=17)
    ap.add_argument("--stop-when-train-acc-gt-test", action="store_true")
    a = ap.parse_args(argv)
    if a.epochs <= 0 or a.batch_size <= 0:
        raise SystemExit("epochs and batch-size must be positive")
    if a.device.startswith("cuda") and not torch.cuda.is_available():
        raise SystemExit("a CUDA device was requested but none is available")
    torch.manual_seed(a.seed)
    device = torch.device(a.device)
    if a.synthetic:
        (xtr, ytr), (xte, yte) = synthetic_split(4096, a.seed), synthetic_split(1024, a.seed + 1)
    else:
        (xtr, ytr), (xte, yte) = load_split(Path(a.data_dir), True), load_split(Path(a.data_dir), False)
    model = Net().to(device)
    params = list(model.parameters())
    opt = Fp32MasterAdamW(params, AdamWOptions(lr=a.lr, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01,
                                               use_master_weights=False))
    csv = open(a.metrics_csv, "w") if a.metrics_csv else None
    if csv:
        csv.write(COLUMNS + "\n")
    print(f"mnist_demo device={device} train_examples={xtr.shape[0]} test_examples={xte.shape[0]} epochs={a.epochs} "
          f"batch_size={a.batch_size} lr={a.lr}", flush=True)
    step, first, last = 0, None, None
    for epoch in range(1, a.epochs + 1):
        model.train()
        order = torch.randperm(xtr.shape[0])
        seen = correct_sum = 0
        loss_sum = 0.0
        for batch, lo in enumerate(range(0, xtr.shape[0], a.batch_size), 1):
            if a.max_train_batches > 0 and batch > a.max_train_batches:
                break
            idx = order[lo:lo + a.batch_size]
            xb, yb = xtr[idx].to(device), ytr[idx].to(device)
            for p in params:
                p.grad = None
            logits = model(xb)
            loss = F.cross_entropy(logits, yb)
            loss.backward()
            opt.step()
            lv, correct = float(loss.detach()), int((logits.argmax(1) == yb).sum())
            first = lv if first is None else first
            last = lv
            step += 1
            loss_sum += lv * xb.shape[0]
            correct_sum += correct
            seen += xb.shape[0]
            if csv:
                csv.write(f"{step},{epoch},{batch},{lv:.8g},{correct / xb.shape[0]:.8g},-1,-1,-1,-1\n")
        tr_loss, tr_acc = evaluate(model, xtr, ytr, device, a.batch_size, a.max_test_batches)
        te_loss, te_acc = evaluate(model, xte, yte, device, a.batch_size, a.max_test_batches)
        print(f"epoch={epoch} steps={step} train_loss={loss_sum / max(seen, 1):.4f} "
              f"train_accuracy={correct_sum / max(seen, 1):.4f} train_eval_accuracy={tr_acc:.4f} "
              f"test_loss={te_loss:.4f} test_accuracy={te_acc:.4f}", flush=True)
        if csv:
            csv.write(f"{step},{epoch},0,{loss_sum / max(seen, 1):.8g},{correct_sum / max(seen, 1):.8g},{tr_loss:.8g},"
                      f"{tr_acc:.8g},{te_loss:.8g},{te_acc:.8g}\n")
        if a.stop_when_train_acc_gt_test and tr_acc > te_acc:
            print(f"stopping: train accuracy {tr_acc:.4f} > test accuracy {te_acc:.4f}", flush=True)
            break
    if csv:
        csv.close()
    if first is None or not (last < first):
        print(f"loss did not fall: first {first} last {last}", file=sys.stderr)
        return 2
    print(f"mnist_demo finished: first_loss={first:.4f} last_loss={last:.4f}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
