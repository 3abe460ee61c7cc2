"""DFlash block-draft speculative decoding, M = 8 rows per verify step."""
from .block import DFlashBlock  # noqa: F401
from .config import DFlashConfig, shrunk_dflash_config  # noqa: F401
from .serve import capture_request, generate_dflash  # noqa: F401
