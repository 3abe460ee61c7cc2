"""Python mirror of the device control block (``enum Ctl`` / ``enum Status`` in csrc/common.cuh).

Like the reference's ``m4_control.py`` / ``m8_control.py`` the header is parsed at import and any
drift between the two descriptions raises (``nex_n2_5_pro/m4_control.py:125-143``).  One 32-word
block serves all three decode modes: BS=1 is the one-row case whose ``(pending, committed_len)``
pair is the reference's ``slot = [token, S]`` (``nex_n2_5_pro/decode_engine.py:22-24``).
"""

from __future__ import annotations

import re
from pathlib import Path

CTL_WORDS = 32
MAX_ROWS = 8


class Ctl:
    COMMITTED_LEN = 0
    STATUS = 1
    COMMIT_COUNT = 2
    PENDING = 3
    IDS = 4
    EMITTED = 12
    ROWS = 20
    FORCED_COMMIT = 21
    STEP_EPOCH = 22
    ACCEPTED = 23
    EOS = 24
    STOP_POS = 25
    FLAGS = 26
    FORCED_SEED = 27
    FORCED_MEAN10 = 28


class Status:
    OK = 0
    REDUCE_TIMEOUT = 1
    NON_FINITE = 2
    BAD_CONFIG = 3
    CP_TIMEOUT = 4
    BAD_TOKEN = 5
    PIPE_TIMEOUT = 6


_HEADER_NAMES = {
    "kCtlCommittedLen": Ctl.COMMITTED_LEN, "kCtlStatus": Ctl.STATUS, "kCtlCommitCount": Ctl.COMMIT_COUNT,
    "kCtlPending": Ctl.PENDING, "kCtlIds": Ctl.IDS, "kCtlEmitted": Ctl.EMITTED, "kCtlRows": Ctl.ROWS,
    "kCtlForcedCommit": Ctl.FORCED_COMMIT, "kCtlStepEpoch": Ctl.STEP_EPOCH, "kCtlAccepted": Ctl.ACCEPTED,
    "kCtlEos": Ctl.EOS, "kCtlStopPos": Ctl.STOP_POS, "kCtlFlags": Ctl.FLAGS, "kCtlForcedSeed": Ctl.FORCED_SEED,
    "kCtlForcedMean10": Ctl.FORCED_MEAN10, "kCtlWords": CTL_WORDS,
    "kStatusOk": Status.OK, "kStatusReduceTimeout": Status.REDUCE_TIMEOUT, "kStatusNonFinite": Status.NON_FINITE,
    "kStatusBadConfig": Status.BAD_CONFIG, "kStatusCpTimeout": Status.CP_TIMEOUT, "kStatusBadToken": Status.BAD_TOKEN,
    "kStatusPipeTimeout": Status.PIPE_TIMEOUT, "kMaxRows": MAX_ROWS,
}


def parse_header(text: str) -> dict:
    found = {}
    for name, value in re.findall(r"\b(k[A-Z]\w+)\s*=\s*(\d+)\s*[,;]", text):
        found[name] = int(value)
    return found


def check_abi(header_path=None) -> None:
    path = Path(header_path) if header_path else Path(__file__).resolve().parent.parent / "csrc" / "common.cuh"
    found = parse_header(path.read_text())
    for name, value in _HEADER_NAMES.items():
        if name not in found:
            raise RuntimeError(f"control ABI drift: {name} missing from {path.name}")
        if found[name] != value:
            raise RuntimeError(f"control ABI drift: {name} is {found[name]} in {path.name}, {value} in Python")


check_abi()


def conv_slot(position: int, ring: int) -> int:
    """History-ring slot of the pre-convolution row of ``position``."""
    return position % ring


def state_slot(position: int, ring: int) -> int:
    """State-ring slot holding the recurrent state BEFORE ``position`` is consumed."""
    return position % ring


def ring_no_alias(rows: int, conv_ring: int, state_ring: int) -> bool:
    """A step of ``rows`` rows never overwrites what its own re-execution reads."""
    return conv_ring >= rows + 3 and state_ring >= rows + 1


def decode_ctl(words) -> dict:
    w = [int(v) for v in words]
    return {
        "committed_len": w[Ctl.COMMITTED_LEN], "status": w[Ctl.STATUS], "commit_count": w[Ctl.COMMIT_COUNT],
        "pending": w[Ctl.PENDING], "ids": w[Ctl.IDS : Ctl.IDS + 8], "emitted": w[Ctl.EMITTED : Ctl.EMITTED + 8],
        "accepted": w[Ctl.ACCEPTED], "step_epoch": w[Ctl.STEP_EPOCH], "stop_pos": w[Ctl.STOP_POS],
    }
