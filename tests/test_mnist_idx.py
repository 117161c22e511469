"""IDX loader: round trip through files written in the format (raw and gzipped), header errors."""
import gzip
import os
import struct

import numpy as np
import pytest
import torch

from mnist_idx import batches, load_mnist, read_idx


def _write_idx(path, arr, gz=False):
    head = bytes([0, 0, 0x08, arr.ndim]) + struct.pack(">" + "I" * arr.ndim, *arr.shape)
    opener = gzip.open if gz else open
    with opener(path, "wb") as f:
        f.write(head + arr.astype(np.uint8).tobytes())


def test_round_trip_raw_and_gz(tmp_path):
    rng = np.random.default_rng(0)
    img = rng.integers(0, 256, size=(37, 28, 28), dtype=np.uint8)
    lab = rng.integers(0, 10, size=(37,), dtype=np.uint8)
    _write_idx(os.path.join(tmp_path, "train-images-idx3-ubyte"), img)
    _write_idx(os.path.join(tmp_path, "train-labels-idx1-ubyte.gz"), lab, gz=True)
    assert np.array_equal(read_idx(os.path.join(tmp_path, "train-images-idx3-ubyte")), img)
    x, y = load_mnist(str(tmp_path), "train", normalize=False)
    assert x.shape == (37, 1, 28, 28) and x.dtype == torch.float32 and y.dtype == torch.int64
    assert torch.equal((x * 255).round().to(torch.uint8).squeeze(1), torch.from_numpy(img))
    assert torch.equal(y, torch.from_numpy(lab).long())
    xn, _ = load_mnist(str(tmp_path), "train")
    assert torch.allclose(xn, (x - 0.1307) / 0.3081)
    seen = sum(b[0].shape[0] for b in batches(x, y, 8, generator=torch.Generator().manual_seed(1)))
    assert seen == 32                                    # 37 // 8 * 8: the ragged tail is dropped
    assert sum(b[0].shape[0] for b in batches(x, y, 8, shuffle=False, drop_last=False)) == 37


def test_bad_files(tmp_path):
    p = os.path.join(tmp_path, "junk")
    open(p, "wb").write(b"\x01\x02\x03\x04rest")
    with pytest.raises(ValueError):
        read_idx(p)
    short = os.path.join(tmp_path, "short")
    open(short, "wb").write(bytes([0, 0, 8, 1]) + struct.pack(">I", 10) + b"123")
    with pytest.raises(ValueError):
        read_idx(short)
    with pytest.raises(FileNotFoundError):
        load_mnist(str(tmp_path), "test")
