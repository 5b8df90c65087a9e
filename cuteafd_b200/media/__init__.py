"""Bundled media towers: image / audio decoding and preprocessing, vision and audio encoders, an embedding cache,
and the processor that turns chat content parts into placeholder tokens plus embedding rows for the engines."""
from .image import decode_image, preprocess_image, smart_resize  # noqa: F401
from .processor import MediaProcessor, MediaSpan  # noqa: F401
from .towers import AudioTower, AudioTowerConfig, VisionTower, VisionTowerConfig  # noqa: F401
