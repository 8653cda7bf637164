"""Constants of the INT8-X scheme (values follow ixrun/config.py:21-51)."""

DEFAULT_LEVELS = (3, 5, 8)
# names that keep their native dtype when a model is deployed
SKIP_PATTERNS = ("lm_head", "embed", "shared", "wte", "wte_emb")
# linears smaller than this stay unquantised
MIN_LINEAR_ELEMS = 1000
# elements per rank block (granularity of the block prefix tables)
RANK_BLOCK = 1024
