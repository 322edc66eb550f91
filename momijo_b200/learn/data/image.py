"""``ImageFolderDataset``: ``root/<class>/<file>`` with PPM/PGM/PNG/JPEG decoding through
``momijo_b200.vision`` (legacy/src/momijo/learn/data/image.mojo:131)."""
from __future__ import annotations

import os

import torch

EXTS = (".ppm", ".pgm", ".png", ".jpg", ".jpeg", ".bmp")


class ImageFolderDataset:
    def __init__(self, root: str, transform=None, as_chw_float: bool = True):
        self.root, self.transform, self.as_chw_float = root, transform, as_chw_float
        self.classes = sorted(d for d in os.listdir(root) if os.path.isdir(os.path.join(root, d)))
        self.class_to_idx = {c: i for i, c in enumerate(self.classes)}
        self.samples = []
        for c in self.classes:
            for f in sorted(os.listdir(os.path.join(root, c))):
                if f.lower().endswith(EXTS):
                    self.samples.append((os.path.join(root, c, f), self.class_to_idx[c]))

    def __len__(self):
        return len(self.samples)

    def num_classes(self) -> int:
        return len(self.classes)

    def class_name(self, idx: int) -> str:
        """Name of class ``idx``; empty for an index outside the class list."""
        return self.classes[idx] if 0 <= idx < len(self.classes) else ""

    def __getitem__(self, i):
        from ...vision import imread

        path, label = self.samples[i]
        img = imread(path)
        if self.transform is not None:
            img = self.transform(img)
        t = img.to_tensor() if hasattr(img, "to_tensor") else torch.as_tensor(img)
        if self.as_chw_float and t.dim() == 3:
            t = t.permute(2, 0, 1).float() / 255.0
        return t, label

    get = __getitem__


def list_dirs_sorted(root: str):
    """Names of the sub-directories of ``root`` in lexicographic order; [] if ``root`` cannot be listed
    (legacy/src/momijo/learn/data/image.mojo:70-91)."""
    try:
        return sorted(d for d in os.listdir(root) if os.path.isdir(os.path.join(root, d)))
    except OSError:
        return []


def list_dirs_sorted_paths(root: str):
    return [os.path.join(root, d) for d in list_dirs_sorted(root)]


def list_pngs_sorted(root: str):
    """Full paths of the ``.png`` files (any case) of ``root``, sorted by file name."""
    try:
        return [os.path.join(root, f) for f in sorted(os.listdir(root)) if f.lower().endswith(".png")]
    except OSError:
        return []
