"""Request states; their integer order is the sort key of the batch assembler
(src/loquetier_src/enums.py:3-6, used at model_generation.py:186,248)."""
from enum import IntEnum


class InferStatus(IntEnum):
    Train = 0
    Prefill = 1
    Decode = 2
