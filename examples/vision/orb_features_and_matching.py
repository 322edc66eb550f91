"""Corner features with binary descriptors, brute-force Hamming matching between an image and a shifted copy
(mirrors legacy/examples/vision/orb_features_and_matching.mojo)."""
import torch

import momijo.vision as V


def main():
    g = torch.Generator().manual_seed(0)
    base = V.Image.new_hwc_u8(96, 96, 1, 0)
    for _ in range(14):
        x, y = int(torch.randint(8, 80, (1,), generator=g)), int(torch.randint(8, 80, (1,), generator=g))
        V.rectangle(base, x, y, x + 9, y + 7, (int(torch.randint(90, 255, (1,), generator=g)),), -1)
    moved = V.Image(torch.roll(base.data, shifts=(3, 5), dims=(0, 1)).contiguous())
    k1, d1 = V.orb_detect_and_compute(base, 80)
    k2, d2 = V.orb_detect_and_compute(moved, 80)
    matches = V.top_k_matches(V.bf_match_hamming(d1, d2), 20)
    shifts = [(V.keypoint_xy(k2, j)[0] - V.keypoint_xy(k1, i)[0], V.keypoint_xy(k2, j)[1] - V.keypoint_xy(k1, i)[1])
              for i, j, _ in matches]
    good = sum(1 for s in shifts if s == (5, 3))
    side = V.draw_matches(V.gray_to_bgr(base), k1, V.gray_to_bgr(moved), k2, matches)
    print("keypoints:", V.len_keypoints(k1), V.len_keypoints(k2), "matches:", len(matches), "with the true shift:", good, side.shape)
    assert len(matches) > 0 and good >= len(matches) // 2
    return side


if __name__ == "__main__":
    main()
