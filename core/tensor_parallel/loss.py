from gpt_from_scratch_b200.parallel.loss import _VocabParallelCrossEntropy, vocab_parallel_cross_entropy  # noqa: F401
