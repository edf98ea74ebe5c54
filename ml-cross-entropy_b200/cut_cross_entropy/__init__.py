"""B200-native Cut Cross-Entropy: the ``cut_cross_entropy`` API over hand-written sm_100a CUDA."""

from .cce_utils import LinearCrossEntropyImpl
from .linear_cross_entropy import LinearCrossEntropy, linear_cross_entropy
from .vocab_parallel import VocabParallelOptions

__all__ = [
    "LinearCrossEntropy",
    "LinearCrossEntropyImpl",
    "linear_cross_entropy",
    "VocabParallelOptions",
]

__version__ = "0.1.0"
