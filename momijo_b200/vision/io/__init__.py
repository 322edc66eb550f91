from .image import (decode_image, encode_image, format_from_path, imread, imwrite, read_image, read_image_any,  # noqa: F401
                    read_jpeg, read_png, read_ppm, register_codec, sniff_format, write_image, write_image_any,
                    write_jpeg, write_png, write_ppm)
from .jpeg import decode_jpeg, encode_jpeg  # noqa: F401
from .png import decode_png, encode_png  # noqa: F401
from .ppm import decode_ppm, encode_ppm  # noqa: F401
