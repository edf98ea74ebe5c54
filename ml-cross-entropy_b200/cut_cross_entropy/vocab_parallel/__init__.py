from .utils import VocabParallelOptions, partition_n_into_range


def vocab_parallel_torch_compile_lce_apply(*args, **kwargs):
    """The reference's materialised-logits vocab-parallel path
    (``cut_cross_entropy/vocab_parallel/vocab_parallel_torch_compile.py``).  Like
    ``impl="torch_compile"`` it is not part of this backend, which has no path that forms the
    ``[N, V]`` logits: call ``linear_cross_entropy(..., vocab_parallel_options=...)`` instead."""
    raise NotImplementedError(
        "the torch_compile (materialised logits) path is not part of the B200 backend; "
        "use linear_cross_entropy(..., impl='cce', vocab_parallel_options=...)"
    )


__all__ = ["VocabParallelOptions", "partition_n_into_range", "vocab_parallel_torch_compile_lce_apply"]
