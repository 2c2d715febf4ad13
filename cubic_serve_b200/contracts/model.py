"""Model-level contracts: what a loaded model needs from the runtime, stated as data.

* ``CacheSpec``  -- the paged KV cache of the full-attention layers: page size, independently typed K and V codes,
  scale groups, bytes per page;
* ``StateSpec``  -- the per-request recurrent state of Gated DeltaNet layers (delta-rule state and causal-conv inputs);
* ``WeightManifest`` -- every tensor of a checkpoint with dtype, shape and shard file, and a digest over that list
  (the operand digest of start-up evidence);
* ``ModelSpec``  -- architecture + cache + state (+ manifest): memory planning (`kv_pages`) and digests come from it.

All sizes are per rank: ``tp`` divides heads, ``layers`` restricts to a pipeline stage.

Reference counterpart: ``contracts/model.py:66-273`` (``ModelSpec``, ``StateSpec``, ``CacheSpec``, ``WeightManifest``).
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass

from .implementation import digest_of

PAGE_TOKENS = 16
KV_SCALE_GROUP = 32          # channels per fp32 scale, for K and for V
GDN_HEAD_DIM = 128
GDN_CONV_TAPS = 4


@dataclass(frozen=True)
class CacheSpec:
    layers: int               # full-attention layers held by this rank
    kv_heads: int             # rank-local key/value heads
    head_dim: int
    k_bits: int
    v_bits: int
    page_tokens: int = PAGE_TOKENS

    def __post_init__(self) -> None:
        for bits in (self.k_bits, self.v_bits):
            if bits not in (4, 6, 8):
                raise ValueError(f"KV codes are 4, 6 or 8 bits wide, not {bits}")
        if self.head_dim % KV_SCALE_GROUP:
            raise ValueError(f"head_dim must be a multiple of the {KV_SCALE_GROUP}-channel scale group")

    @property
    def blob_bytes(self) -> int:
        """One (page, kv head) blob: K codes, K scales, V codes, V scales (``csrc/kv_layout.cuh``)."""
        codes = self.page_tokens * self.head_dim * (self.k_bits + self.v_bits) // 8
        scales = 2 * self.page_tokens * (self.head_dim // KV_SCALE_GROUP) * 4
        return codes + scales

    @property
    def page_bytes(self) -> int:
        """One page across all local layers and heads."""
        return self.layers * self.kv_heads * self.blob_bytes

    def bytes_per_token(self) -> float:
        return self.page_bytes / self.page_tokens


@dataclass(frozen=True)
class StateSpec:
    layers: int               # Gated DeltaNet layers held by this rank
    k_heads: int              # rank-local key heads
    v_heads: int              # rank-local value heads

    @property
    def delta_bytes(self) -> int:
        """fp32 ``[v_heads, 128, 128]`` delta-rule state of one request in one layer."""
        return self.v_heads * GDN_HEAD_DIM * GDN_HEAD_DIM * 4

    @property
    def conv_bytes(self) -> int:
        """bf16 inputs of the last ``taps - 1`` positions over the q | k | v channels."""
        return (GDN_CONV_TAPS - 1) * (2 * self.k_heads + self.v_heads) * GDN_HEAD_DIM * 2

    @property
    def bytes_per_request(self) -> int:
        return self.layers * (self.delta_bytes + self.conv_bytes)


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: str
    shape: tuple[int, ...]
    file: str


@dataclass(frozen=True)
class WeightManifest:
    tensors: tuple[TensorEntry, ...]

    @staticmethod
    def from_store(store) -> "WeightManifest":
        """From a ``models.checkpoint.SafetensorsDirectory`` (headers only, no tensor data is read)."""
        return WeightManifest(tuple(TensorEntry(t.name, t.dtype, tuple(t.shape), t.file)
                                    for t in sorted(store.tensors.values(), key=lambda t: t.name)))

    @property
    def digest(self) -> str:
        return digest_of([[t.name, t.dtype, list(t.shape), t.file] for t in self.tensors])

    @property
    def files(self) -> tuple[str, ...]:
        return tuple(sorted({t.file for t in self.tensors}))

    def __len__(self) -> int:
        return len(self.tensors)


@dataclass(frozen=True)
class ModelSpec:
    name: str
    family: str
    config_digest: str
    cache: CacheSpec
    state: StateSpec | None
    manifest: WeightManifest | None = None

    @staticmethod
    def from_config(cfg, k_bits: int = 8, v_bits: int = 8, tp: int = 1, layers: tuple[int, int] | None = None,
                    manifest: WeightManifest | None = None) -> "ModelSpec":
        lo, hi = layers or (0, cfg.num_layers)
        n_gdn = sum(cfg.layer_is_gdn(i) for i in range(lo, hi))
        from ..models.config import kv_heads_of_rank
        kv_local = kv_heads_of_rank(cfg.num_kv_heads, 0, tp)[1]       # a head shared by several ranks is cached on each
        cache = CacheSpec(hi - lo - n_gdn, kv_local, cfg.head_dim, k_bits, v_bits)
        state = StateSpec(n_gdn, cfg.gdn_k_heads // tp, cfg.gdn_v_heads // tp) if n_gdn else None
        return ModelSpec(cfg.name, cfg.family, digest_of(dataclasses.asdict(cfg)), cache, state, manifest)

    @property
    def digest(self) -> str:
        """Operand digest of this model for start-up evidence: architecture, cache typing and the tensor manifest."""
        return digest_of({"config": self.config_digest, "cache": dataclasses.asdict(self.cache),
                          "state": None if self.state is None else dataclasses.asdict(self.state),
                          "manifest": None if self.manifest is None else self.manifest.digest})

    def kv_pages(self, free_bytes: int, reserve_bytes: int, max_model_len: int, max_running: int,
                 state_snapshots: int = 0) -> int:
        """Pages that fit into what is left of the device after the reserve and the recurrent state of
        ``max_running`` requests (plus ``state_snapshots`` snapshot rows kept for cached prefixes), capped by what
        ``max_running`` requests of ``max_model_len`` tokens can use."""
        budget = max(0, free_bytes - reserve_bytes)
        if self.state is not None:
            budget = max(0, budget - (max_running + state_snapshots) * self.state.bytes_per_request)
        cap = max_running * (-(-max_model_len // self.cache.page_tokens)) + 64
        if self.cache.page_bytes == 0:                 # a stage without full-attention layers still needs page ids
            return int(cap)
        return int(max(64, min(budget // self.cache.page_bytes, cap)))
