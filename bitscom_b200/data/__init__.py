"""Input pipeline of the trainers: tokenizers that need no download, text and packed-token
datasets, a deterministic data-parallel sampler and a prefetching loader that hands out
pinned host batches."""

from .dataset import (DistributedBatchSampler, PackedTokenDataset, TextLineDataset,  # noqa: F401
                      tokenize_to_file)
from .loader import PrefetchLoader, SyntheticTokens, build_loader  # noqa: F401
from .tokenizer import ByteTokenizer, SentencePieceTokenizer, load_tokenizer  # noqa: F401
