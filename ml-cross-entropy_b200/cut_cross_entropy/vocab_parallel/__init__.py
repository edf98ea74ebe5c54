from .utils import VocabParallelOptions, partition_n_into_range

__all__ = ["VocabParallelOptions", "partition_n_into_range"]
