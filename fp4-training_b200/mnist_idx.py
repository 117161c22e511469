"""Loader for the MNIST IDX files (the reference's training script downloads them through
torchvision, main_train_tinyvit_mnist.py:46-47; here they are read from a local directory, raw
or gzipped, without torchvision).

IDX format: big-endian header `00 00 <type> <ndim>` followed by ndim uint32 extents and the
data in row-major order; type 0x08 is unsigned byte (the four MNIST files use only that)."""
from __future__ import annotations

import gzip
import os
import struct

import numpy as np
import torch

_DTYPES = {0x08: np.uint8, 0x09: np.int8, 0x0B: ">i2", 0x0C: ">i4", 0x0D: ">f4", 0x0E: ">f8"}
FILES = {
    "train": ("train-images-idx3-ubyte", "train-labels-idx1-ubyte"),
    "test": ("t10k-images-idx3-ubyte", "t10k-labels-idx1-ubyte"),
}
MEAN, STD = 0.1307, 0.3081      # the normalisation the reference applies (main_train_tinyvit_mnist.py:42-45)


def read_idx(path: str) -> np.ndarray:
    """One IDX file (optionally .gz) -> numpy array of its declared shape."""
    opener = gzip.open if path.endswith(".gz") else open
    with opener(path, "rb") as f:
        head = f.read(4)
        if len(head) != 4 or head[0] != 0 or head[1] != 0:
            raise ValueError(f"{path}: not an IDX file (bad magic {head!r})")
        code, ndim = head[2], head[3]
        if code not in _DTYPES:
            raise ValueError(f"{path}: unknown IDX element type 0x{code:02x}")
        raw_dims = f.read(4 * ndim)
        if len(raw_dims) != 4 * ndim:
            raise ValueError(f"{path}: truncated header")
        dims = struct.unpack(">" + "I" * ndim, raw_dims)
        dt = np.dtype(_DTYPES[code])
        count = int(np.prod(dims)) if dims else 1
        data = f.read(count * dt.itemsize)
        if len(data) != count * dt.itemsize:
            raise ValueError(f"{path}: expected {count} elements, file holds {len(data) // dt.itemsize}")
    return np.frombuffer(data, dtype=dt).reshape(dims)


def _find(root: str, stem: str) -> str:
    for cand in (stem, stem + ".gz", stem.replace("-idx", ".idx"), stem.replace("-idx", ".idx") + ".gz"):
        p = os.path.join(root, cand)
        if os.path.isfile(p):
            return p
    raise FileNotFoundError(f"{stem}[.gz] not found in {root}")


def load_mnist(root: str, split: str = "train", normalize: bool = True, device="cpu"):
    """-> (images float32 [N, 1, 28, 28], labels int64 [N]); images scaled to [0, 1] and, with
    normalize, standardised with the reference's mean / std."""
    img_name, lab_name = FILES[split]
    images = read_idx(_find(root, img_name))
    labels = read_idx(_find(root, lab_name))
    if images.ndim != 3 or labels.ndim != 1 or images.shape[0] != labels.shape[0]:
        raise ValueError(f"unexpected shapes: images {images.shape}, labels {labels.shape}")
    x = torch.from_numpy(images.copy()).to(torch.float32).div_(255.0).unsqueeze(1)
    if normalize:
        x = (x - MEAN) / STD
    return x.to(device), torch.from_numpy(labels.copy()).to(torch.int64).to(device)


def batches(x: torch.Tensor, y: torch.Tensor, batch_size: int, shuffle: bool = True, generator=None, drop_last=True):
    """Mini-batch iterator over tensors already on their device."""
    n = x.shape[0]
    order = torch.randperm(n, generator=generator, device="cpu") if shuffle else torch.arange(n)
    stop = n - n % batch_size if drop_last else n
    for i in range(0, stop, batch_size):
        idx = order[i:i + batch_size].to(x.device)
        yield x[idx], y[idx]
