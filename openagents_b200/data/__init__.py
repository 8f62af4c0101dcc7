"""Training data: token shards, the shuffled sampler and prefetching loader (C++), byte-level BPE (C++), the text
refinery and the conversions from chat records and session traces to supervised examples."""
from .shards import BatchLoader, TokenDataset, permute, write_token_shard  # noqa: F401
from .bpe import ByteBpe  # noqa: F401
