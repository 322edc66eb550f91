from .image import (decode_image, encode_image, format_from_path, imread, imwrite, read_image, read_image_any,  # noqa: F401
                    read_jpeg, read_png, read_ppm, register_codec, sniff_format, write_image, write_image_any,
                    write_jpeg, write_png, write_ppm)
from .jpeg import decode_jpeg, encode_jpeg  # noqa: F401
from .png import decode_png, encode_png  # noqa: F401
from .ppm import decode_ppm, encode_ppm  # noqa: F401
from . import deflate, file_io, jpeg_parts  # noqa: F401,E402
from .deflate import (CLE, HC, Huff, Huffman, Tok, adler32, crc32, deflate_dynamic_stream, deflate_fixed_stream,  # noqa: F401,E402
                      make_lit, make_match, put_code, zlib_deflate, zlib_inflate, zlib_stored)
from .file_io import (MemFileStore, ensure_outdir, memfs_append_ptr, memfs_clear_all, memfs_ensure_path,  # noqa: F401,E402
                      memfs_has_path, memfs_list_all, memfs_remove_path, memfs_size_of, memfs_try_read,
                      memfs_write_replace, read_all_bytes, write_all_bytes)
from .image import (has_jpeg_codec, make_dummy_u8_hwc_tensor, read_image_auto, read_image_auto_with_fallback,  # noqa: F401,E402
                    read_image_with_fallback, read_jpeg_image, read_jpeg_with_fallback, unsafe_char_from_code,
                    write_jpeg_image)
from .jpeg_parts import *  # noqa: F401,F403,E402
from .png import (PNGChunk, PNGHeader, debug_sample_rgb, decode_png_bytes, decode_png_bytes_u16, is_png_magic,  # noqa: F401,E402
                  parse_chunk, parse_ihdr, parse_png_header, png_from_hwc_u8, png_unfilter, read_be_u32,
                  read_png_header_only, read_png_u16_raw)
