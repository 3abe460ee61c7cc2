"""Native multi-token-prediction (MTP) speculative decoding, M = 4 rows per verify step."""
from .block import MtpDraft  # noqa: F401
from .serve import capture_round, generate_mtp  # noqa: F401
