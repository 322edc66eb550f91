from .array import *  # noqa: F401,F403
from .bitwise import bitwise_and, bitwise_not, bitwise_or  # noqa: F401
from .color import (bgr_to_gray, bgr_to_rgb, clahe_color_bgr, color_jitter, equalize_hist, gray_to_bgr,  # noqa: F401
                    histogram, merge3, plot_hist_u8, rgb_to_bgr, rgb_to_gray, split3)
from .compose import (Compose, Normalize, Step, StepAffine, StepNorm, build_transforms, make_step_affine,  # noqa: F401
                      make_step_norm, normalize, normalize_chw, to_tensor)
from .contour import (arc_length, bounding_rect, contour_area, find_contours, get_contour, is_on_u8,  # noqa: F401
                      len_contours)
from .draw import (Int32Mat, arrowed_line, as_u8, bgr_u8, circle, draw_circles, draw_contours, draw_lines_p,  # noqa: F401
                   draw_matches, fill_poly, label_to_color, label_to_color_image, line, put_text, rectangle)
from .filter import (bilateral_blur, bilateral_filter, canny, gaussian_blur, laplacian, magnitude_u8,  # noqa: F401
                     median_blur, ones_u8, sobel)
from .geom import *  # noqa: F401,F403
from .hough import hough_circles, hough_lines, hough_lines_p  # noqa: F401
from .morph import MORPH_DILATE, MORPH_ERODE, dilate, erode, morphology  # noqa: F401
from .segmentation import connected_components  # noqa: F401
from .threshold import adaptive_threshold, otsu_level, threshold_binary, threshold_otsu  # noqa: F401
from .random_ops import (ColorJitter, Keypoint, RandomHorizontalFlip, RandomResizedCrop, RandomRotation,  # noqa: F401,E402
                         ToTensor, abs_f64, maybe_resize_placeholder, random_affine_placeholder,
                         random_resized_crop, resize_nearest_u8_hwc, resize_nearest_u8_hwc_tiled,
                         resize_nearest_u8_hwc_tiled_scheduled)
