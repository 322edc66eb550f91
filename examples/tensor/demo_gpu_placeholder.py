"""Device query and a device round trip (runs on the CPU when no GPU is present)
(legacy/examples/tensor/demo_gpu_placeholder.mojo)."""
import numpy as np

import momijo.tensor as mt


def main():
    import torch
    has = mt.gpu_available()
    assert has == torch.cuda.is_available()
    t = mt.arange_f32(0, 8)
    if has:
        d = t.cuda()
        assert (d * 2).cpu().tolist() == (t * 2).tolist()
    moved = mt.to_device(t, mt.Device.gpu() if has else mt.Device.cpu())   # falls back to the CPU without a GPU
    assert moved.cpu().tolist() == t.tolist()
    print("gpu available:", has)
    return has is not None


if __name__ == "__main__":
    main()
