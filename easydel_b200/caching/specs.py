"""What each kind of layer has to keep in the serving cache, and how a memory budget is divided between them.

Role of easydel/caching/_specs.py:82-531 (``KVCacheSpec`` and its ``FullAttentionSpec`` / ``SlidingWindowSpec`` /
``ChunkedLocalAttentionSpec`` / ``MambaSpec`` / ``MLAAttentionSpec`` subclasses with their ``page_size_bytes`` and
``max_memory_usage_bytes``) and of the grouping step of the reference's cache coordinator
(easydel/inference/esurge/core/kv_cache_coordinator.py): layers that retain keys under the same rule form one
*group* with its own page pool and page tables; a group of sliding-window or chunked-local layers never needs more
pages than its window covers, whatever the sequence length, and the rest of the memory goes to the full-attention
group.
"""

from __future__ import annotations

from dataclasses import dataclass, field

PAGE_TOKENS = 128


def cdiv(a: int, b: int) -> int:
    return -(-a // b)


@dataclass(frozen=True)
class KVCacheSpec:
    """Keys + values of one layer in pages of ``page_size`` tokens."""

    page_size: int = PAGE_TOKENS
    num_kv_heads: int = 1
    head_dim: int = 128
    element_size: int = 2
    kind: str = "full"

    @property
    def page_size_bytes(self) -> int:
        return 2 * self.page_size * self.num_kv_heads * self.head_dim * self.element_size

    def tokens_kept(self, context: int) -> int:
        return context

    def first_useful_token(self, num_computed_tokens: int) -> int:
        """Keys before this position are never read again once ``num_computed_tokens`` tokens are in the cache."""
        return 0

    def pages_per_sequence(self, max_model_len: int, max_step_tokens: int = 1) -> int:
        """Upper bound of pages one sequence holds (``max_step_tokens`` new tokens are appended before old pages are
        released)."""
        return cdiv(max_model_len, self.page_size)

    def max_memory_usage_bytes(self, max_model_len: int, max_step_tokens: int = 1) -> int:
        return self.pages_per_sequence(max_model_len, max_step_tokens) * self.page_size_bytes

    def group_key(self) -> tuple:
        return (self.kind, 0, self.num_kv_heads, self.head_dim, self.element_size)


@dataclass(frozen=True)
class FullAttentionSpec(KVCacheSpec):
    kind: str = "full"


@dataclass(frozen=True)
class SlidingWindowSpec(KVCacheSpec):
    sliding_window: int = 4096
    kind: str = "sliding"

    def tokens_kept(self, context: int) -> int:
        return min(context, self.sliding_window)

    def first_useful_token(self, num_computed_tokens: int) -> int:
        # the next query sits at position num_computed_tokens and sees keys > position - window
        return max(0, num_computed_tokens - self.sliding_window + 1)

    def pages_per_sequence(self, max_model_len: int, max_step_tokens: int = 1) -> int:
        span = min(max_model_len, self.sliding_window - 1 + max_step_tokens)
        return min(cdiv(max_model_len, self.page_size), cdiv(span, self.page_size) + 1)

    def group_key(self) -> tuple:
        return (self.kind, self.sliding_window, self.num_kv_heads, self.head_dim, self.element_size)


@dataclass(frozen=True)
class ChunkedLocalAttentionSpec(KVCacheSpec):
    attention_chunk_size: int = 8192
    kind: str = "chunked"

    def tokens_kept(self, context: int) -> int:
        return min(context, self.attention_chunk_size)

    def first_useful_token(self, num_computed_tokens: int) -> int:
        # a query only sees the keys of its own block of ``attention_chunk_size`` positions
        return (num_computed_tokens // self.attention_chunk_size) * self.attention_chunk_size

    def pages_per_sequence(self, max_model_len: int, max_step_tokens: int = 1) -> int:
        span = min(max_model_len, self.attention_chunk_size + max_step_tokens)
        return min(cdiv(max_model_len, self.page_size), cdiv(span, self.page_size) + 1)

    def group_key(self) -> tuple:
        return (self.kind, self.attention_chunk_size, self.num_kv_heads, self.head_dim, self.element_size)


@dataclass(frozen=True)
class MLAAttentionSpec(KVCacheSpec):
    """One row ``[latent | rotary key]`` per token, shared by every head; no separate value pool."""

    kind: str = "latent"

    @property
    def page_size_bytes(self) -> int:
        return self.page_size * self.num_kv_heads * self.head_dim * self.element_size


@dataclass(frozen=True)
class MambaSpec(KVCacheSpec):
    """A fixed-size state per sequence (SSM, delta rule, lightning attention): one "page" per sequence."""

    state_elements: int = 0
    kind: str = "recurrent"

    @property
    def page_size_bytes(self) -> int:
        return self.state_elements * self.element_size

    def tokens_kept(self, context: int) -> int:
        return 0

    def pages_per_sequence(self, max_model_len: int, max_step_tokens: int = 1) -> int:
        return 1


@dataclass
class KVCacheGroup:
    spec: KVCacheSpec
    layers: list[int] = field(default_factory=list)
    num_pages: int = 0

    @property
    def kind(self) -> str:
        return self.spec.kind

    @property
    def window(self) -> int:
        return getattr(self.spec, "sliding_window", 0) or getattr(self.spec, "attention_chunk_size", 0)

    @property
    def bytes_per_page(self) -> int:
        return self.spec.page_size_bytes * len(self.layers)


def layer_spec(info, element_size: int = 2, tp_size: int = 1, page_size: int = PAGE_TOKENS) -> KVCacheSpec | None:
    """Spec of one layer from its :class:`~easydel_b200.infra.mixins.operation_cache.LayerOperationInfo`."""
    if not info.requires_kv_cache:
        return None
    kvh = max(1, info.num_kv_heads // max(1, tp_size)) if info.layer_type != "latent_attention" else 1
    common = dict(page_size=page_size, num_kv_heads=kvh, head_dim=info.head_dim, element_size=element_size)
    if info.layer_type == "latent_attention":
        return MLAAttentionSpec(**common)
    if info.sliding_window:
        return SlidingWindowSpec(sliding_window=int(info.sliding_window), **common)
    if info.chunk_size:
        return ChunkedLocalAttentionSpec(attention_chunk_size=int(info.chunk_size), **common)
    return FullAttentionSpec(**common)


def build_groups(model, element_size: int = 2, tp_size: int = 1, page_size: int = PAGE_TOKENS) -> list[KVCacheGroup]:
    """Groups of layers with the same retention rule and page shape, the full-attention (or latent) group first."""
    info = model.get_operations_cache_info()
    groups: dict[tuple, KVCacheGroup] = {}
    for l in info.layers:
        spec = layer_spec(l, element_size, tp_size, page_size)
        if spec is None:
            continue
        groups.setdefault(spec.group_key(), KVCacheGroup(spec)).layers.append(l.layer_index)
    order = {"full": 0, "latent": 0, "sliding": 1, "chunked": 2}
    return sorted(groups.values(), key=lambda g: (order.get(g.kind, 3), g.window, g.layers[0]))


def plan_pages(groups: list[KVCacheGroup], budget_bytes: int, max_num_seqs: int, max_model_len: int,
               max_num_batched_tokens: int, prefix_cache_slack: float = 0.25) -> list[int]:
    """Pages per group for a memory budget.

    Window-bounded groups get what ``max_num_seqs`` running sequences can ever hold at once — per sequence the pages
    its window covers plus one for the ragged start, plus the pages one step's new tokens can add over the whole
    batch — and a slack share so that released pages stay findable by the prefix cache for a while. Unbounded groups
    share what is left in proportion to their bytes per page (they fill at the same rate); each group's count is
    capped by what ``max_num_seqs`` sequences of ``max_model_len`` tokens need. One extra page per group is the
    null page."""
    P = groups[0].spec.page_size if groups else PAGE_TOKENS
    full_cap = max_num_seqs * cdiv(max_model_len, P) + 1
    out = [0] * len(groups)
    left = int(budget_bytes)
    unbounded = []
    for i, g in enumerate(groups):
        if g.kind in ("sliding", "chunked"):
            per_seq = g.spec.pages_per_sequence(max_model_len, 1)
            need = max_num_seqs * per_seq + cdiv(max_num_batched_tokens, P) + 1
            need = min(full_cap, int(need * (1.0 + prefix_cache_slack)) + 1)
            out[i] = need
            left -= need * g.bytes_per_page
        else:
            unbounded.append(i)
    if unbounded:
        per_page_all = sum(groups[i].bytes_per_page for i in unbounded)
        n = max(2, left // max(1, per_page_all))
        for i in unbounded:
            out[i] = int(min(full_cap, n))
    elif left > 0 and groups:
        # only window-bounded layers: spend the rest on them too (a larger prefix cache)
        per_page_all = sum(g.bytes_per_page for g in groups)
        extra = left // max(1, per_page_all)
        out = [int(min(full_cap, n + extra)) for n in out]
    return [max(2, n) for n in out]
