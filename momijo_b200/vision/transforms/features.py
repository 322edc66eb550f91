"""Keypoints, descriptors and matching (legacy/src/momijo/vision/transforms/features.mojo)."""
from .array import (Descriptor, bf_match_hamming, keypoint_xy, len_keypoints, orb_detect_and_compute,  # noqa: F401
                    to_int_triples, top_k_matches, valid_descriptors)
