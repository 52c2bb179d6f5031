"""Seeded synthetic inputs that stand in for the datasets the reference trains on (CIFAR-10, ImageNet:
neither is available offline).  NumPy PCG64 streams: identical on every platform, so the CPU fixtures, the
GPU tests and the benchmark all see the same bits for a given seed."""
from __future__ import annotations

import numpy as np


def image_batch(batch: int, height: int, classes: int, seed: int):
    """images ~ N(0,1) [B,3,H,H] float32 (normalised-image statistics), labels uniform over `classes`."""
    rng = np.random.default_rng(seed + 7)
    images = rng.standard_normal((batch, 3, height, height)).astype(np.float32)
    labels = rng.integers(0, classes, size=(batch,)).astype(np.int64)
    return images, labels


def resnet20_batch(batch: int, seed: int):
    """CIFAR-shaped batch: [B,3,32,32], 10 classes."""
    return image_batch(batch, 32, 10, seed)
