"""Options of the engine itself (not of a model): cache geometry, batch limits, compute dtype."""
from dataclasses import dataclass

from ..errors import ConfigError


@dataclass(frozen=True)
class EngineConfig:
    dtype: str = "bfloat16"            # "bfloat16": the kernels serving uses; "float32": everything in true 32-bit
    page_size: int = 16                # tokens per cache page
    num_pages: int = 0                 # pages per cache group; 0 = sized from max_tokens
    max_tokens: int = 0                # tokens the cache pool holds when num_pages is 0
    max_requests: int = 8              # live requests (rows of the block table, state slots)
    max_tokens_per_step: int = 2048    # token budget of one step (decode tokens first, then prompt portions)
    chunk: int = 2048                  # most prompt tokens of one request in one step
    max_context: int = 0               # most tokens of one request (prompt + new); 0 = what the pool holds
    cuda_graphs: bool = True           # capture a step shape that comes a second time and replay it from then on
    device: str = "cuda:0"

    def __post_init__(self):
        if self.dtype not in ("bfloat16", "float32"):
            raise ConfigError(f"dtype {self.dtype!r}: bfloat16 or float32")
        if self.page_size < 1:
            raise ConfigError("page_size must be 1 or more")
        if self.max_requests < 1 or self.chunk < 1 or self.max_tokens_per_step < 1:
            raise ConfigError("max_requests, chunk and max_tokens_per_step must be 1 or more")

    def pages(self) -> int:
        if self.num_pages:
            return self.num_pages
        if self.max_tokens:
            return -(-self.max_tokens // self.page_size)
        raise ConfigError("give num_pages or max_tokens")
