"""Step-level execution contracts: what a batch is, which state it may touch, what a speculative round commits,
which operators a sealed execution plan is made of.

Same role as the second half of the reference's ``contracts/execution.py`` (``PlanSegment`` / ``StateTxn`` /
``BatchPlan`` ``:460-755``, ``SpeculativeIteration`` ``:612-715``, ``OpSignature`` ``:985``, ``ExecutionPlan``
``:1847``, the evidence seals ``:1255-1845``), written for this engine: frozen dataclasses that validate on
construction, canonical JSON, SHA-256 seals.  The scheduler's plans (``runtime/scheduler.py::BatchPlan``) are the
mutable working form; ``describe_plan`` turns one into the immutable contract that a trace, a worker command or an
audit can carry, and ``SpeculativeIteration`` is the single place that says which tokens of a draft round are
emitted, committed to the target state and publishable as a prefix.
"""
from __future__ import annotations

import enum
import hashlib
import json
from dataclasses import asdict, dataclass, field


class BatchPhase(str, enum.Enum):
    PREFILL = "prefill"
    DECODE = "decode"
    MIXED = "mixed"
    REVIEW = "review"          # target pass over [root, drafts] of a speculative round


def _digest(payload) -> str:
    return hashlib.sha256(json.dumps(payload, sort_keys=True, separators=(",", ":"), default=str).encode()).hexdigest()


# ------------------------------------------------------------------ segments and state
@dataclass(frozen=True)
class PlanSegment:
    """One request's rows of a step: ``token_count`` tokens from position ``token_start``, written to ``cache_pages``."""
    request_id: str
    phase: BatchPhase
    produces_output: bool
    token_start: int
    token_count: int
    cache_pages: tuple[int, ...]
    state_slot: int = -1                 # row of per-request recurrent state / page-table row, -1 = none

    def __post_init__(self) -> None:
        if not self.request_id:
            raise ValueError("a segment needs a request id")
        if self.token_start < 0 or self.token_count <= 0:
            raise ValueError("a segment covers a positive number of tokens from a non-negative position")
        need = -(-(self.token_start + self.token_count) // 16)
        if len(self.cache_pages) < need:
            raise ValueError(f"segment of {self.request_id} reaches position {self.token_start + self.token_count} "
                             f"but holds {len(self.cache_pages)} pages")
        if any(p < 0 for p in self.cache_pages) or len(set(self.cache_pages)) != len(self.cache_pages):
            raise ValueError("cache pages must be distinct non-negative ids")
        if self.phase is BatchPhase.DECODE and self.token_count != 1:
            raise ValueError("a decode segment has exactly one token")


@dataclass(frozen=True)
class StateAccess:
    """Pages / state slots of one resource (``kv``, ``gdn_state``, ``conv_state``) on one owner rank."""
    resource_id: str
    owner_rank: int
    slots: tuple[int, ...] = ()
    pages: tuple[int, ...] = ()

    def __post_init__(self) -> None:
        if not self.resource_id or self.owner_rank < 0:
            raise ValueError("state access needs a resource and an owner rank")
        if not self.slots and not self.pages:
            raise ValueError("state access names at least one slot or page")


@dataclass(frozen=True)
class PrefixPublishPlan:
    """Which leading tokens of a request become shareable after the step, and from where they would be replayed."""
    prefix_token_count: int
    state_commit_position: int
    commit_alignment_tokens: int = 16

    def __post_init__(self) -> None:
        if self.prefix_token_count < 0 or self.commit_alignment_tokens <= 0:
            raise ValueError("invalid prefix publication")
        if self.prefix_token_count % self.commit_alignment_tokens:
            raise ValueError("a published prefix ends on a page boundary")
        if self.state_commit_position < self.prefix_token_count:
            raise ValueError("state cannot be committed before the prefix it covers")

    @property
    def replay_token_count(self) -> int:
        """Tokens between the published boundary and the committed state (recomputed by a request that resumes)."""
        return self.state_commit_position - self.prefix_token_count


@dataclass(frozen=True)
class StateTxn:
    """Copy-on-write transaction of one request's step: revision n -> n + 1, disjoint read / write sets per resource."""
    transaction_id: str
    request_id: str
    base_revision: int
    target_revision: int
    reads: tuple[StateAccess, ...]
    writes: tuple[StateAccess, ...]
    prefix_publish: PrefixPublishPlan | None = None

    def __post_init__(self) -> None:
        if self.target_revision != self.base_revision + 1 or self.base_revision < 0:
            raise ValueError("a transaction advances the request's state by exactly one revision")
        if not self.writes:
            raise ValueError("a transaction writes something")
        for w in self.writes:
            # a page may be read and appended to by its sole owner; state SLOTS are copy-on-write: never both
            for r in self.reads:
                if (r.resource_id, r.owner_rank) == (w.resource_id, w.owner_rank) and set(r.slots) & set(w.slots):
                    raise ValueError(f"transaction {self.transaction_id} reads and writes slot(s) "
                                     f"{sorted(set(r.slots) & set(w.slots))} of {w.resource_id}")


# ------------------------------------------------------------------ speculative rounds
@dataclass(frozen=True)
class SpeculativeIteration:
    """One speculative decision at a target-computed state boundary (reference ``contracts/execution.py:612``).

    The target state holds exactly the first ``target_state_token_count`` tokens.  ``root_token_id`` is the token
    sampled by the previous step: possibly emitted already, not yet processed by the target.  The review pass runs
    ``[root, *drafts]``; the replacement (or, with every draft accepted, the bonus) token is emitted by this
    iteration and becomes the next root, so it is NOT part of the committed target state nor of any published prefix.
    """
    target_state_token_count: int
    root_token_id: int
    draft_token_ids: tuple[int, ...]
    accepted_draft_count: int
    replacement_token_id: int

    def __post_init__(self) -> None:
        if self.target_state_token_count < 0:
            raise ValueError("target state token count must be non-negative")
        if not isinstance(self.draft_token_ids, tuple):
            raise TypeError("draft tokens must be an immutable tuple")
        if any((not isinstance(t, int)) or t < 0 for t in (*self.verify_token_ids, self.replacement_token_id)):
            raise ValueError("token ids must be non-negative integers")
        if not 0 <= self.accepted_draft_count <= len(self.draft_token_ids):
            raise ValueError("accepted draft count must fall within the proposed span")

    @property
    def verify_token_ids(self) -> tuple[int, ...]:
        return (self.root_token_id, *self.draft_token_ids)

    @property
    def committed_target_token_ids(self) -> tuple[int, ...]:
        return (self.root_token_id, *self.draft_token_ids[:self.accepted_draft_count])

    @property
    def committed_target_row_count(self) -> int:
        """Review rows whose KV / recurrent state is kept: the root always is."""
        return self.accepted_draft_count + 1

    @property
    def target_commit_token_count(self) -> int:
        return self.target_state_token_count + self.committed_target_row_count

    @property
    def emitted_token_ids(self) -> tuple[int, ...]:
        """New client-visible tokens (the root was emitted by the round before)."""
        return (*self.draft_token_ids[:self.accepted_draft_count], self.replacement_token_id)

    @property
    def next_root_token_id(self) -> int:
        return self.replacement_token_id

    def prefix_checkpoint_boundary(self, block_size_tokens: int, available_target_boundaries: tuple[int, ...]) -> int | None:
        """Greatest complete-page boundary at or below the committed state for which a recurrent-state checkpoint was
        kept; None = nothing may be published (never KV of one boundary with state of another)."""
        if block_size_tokens <= 0:
            raise ValueError("block size must be positive")
        boundary = self.target_commit_token_count - self.target_commit_token_count % block_size_tokens
        return boundary if boundary and boundary in available_target_boundaries else None


# ------------------------------------------------------------------ batches
@dataclass(frozen=True)
class BatchContract:
    """Immutable description of one planned step."""
    plan_id: str
    phase: BatchPhase
    segments: tuple[PlanSegment, ...]
    logical_rows: int
    capacity_rows: int                   # rows of the graph bucket the step replays (== logical for eager steps)
    topology_id: str
    state_transactions: tuple[StateTxn, ...] = ()
    page_copies: tuple[tuple[int, int], ...] = ()

    def __post_init__(self) -> None:
        if not self.segments:
            raise ValueError("a batch has at least one segment")
        ids = [s.request_id for s in self.segments]
        if len(set(ids)) != len(ids):
            raise ValueError("a request appears once per batch")
        if self.logical_rows != sum(s.token_count for s in self.segments):
            raise ValueError("logical rows must equal the segments' tokens")
        if self.capacity_rows < self.logical_rows:
            raise ValueError("a bucket must hold the batch")
        written: dict[int, str] = {}
        for s in self.segments:
            first = s.token_start // 16
            last = (s.token_start + s.token_count - 1) // 16
            for p in s.cache_pages[first:last + 1]:
                if written.setdefault(p, s.request_id) != s.request_id:
                    raise ValueError(f"page {p} is written by two requests in one step")
        txn_requests = {t.request_id for t in self.state_transactions}
        if txn_requests - set(ids):
            raise ValueError("state transaction of a request that is not in the batch")

    @property
    def padding_rows(self) -> int:
        return self.capacity_rows - self.logical_rows

    def digest(self) -> str:
        return _digest(asdict(self))


def describe_plan(plan, plan_id: str, topology_id: str = "single", capacity_rows: int | None = None) -> BatchContract:
    """The immutable contract of a scheduler plan (``runtime/scheduler.py::BatchPlan``)."""
    segs = []
    for s in plan.segments:
        r = s.request
        phase = BatchPhase.DECODE if s.count == 1 and s.sample and r.output else BatchPhase.PREFILL
        segs.append(PlanSegment(r.request_id, phase, bool(s.sample), s.start, s.count, tuple(r.pages), r.slot))
    rows = sum(s.token_count for s in segs)
    phases = {s.phase for s in segs}
    phase = phases.pop() if len(phases) == 1 else BatchPhase.MIXED
    return BatchContract(plan_id, phase, tuple(segs), rows, capacity_rows or rows, topology_id,
                         page_copies=tuple((int(a), int(b)) for a, b in plan.copies))


# ------------------------------------------------------------------ operators and execution plans
@dataclass(frozen=True)
class TensorSpec:
    name: str
    dtype: str
    shape: tuple                         # ints or symbol names

    def __post_init__(self) -> None:
        if not self.name.isidentifier():
            raise ValueError("tensor names are identifiers")
        if any(not isinstance(d, (int, str)) or (isinstance(d, int) and d <= 0) for d in self.shape):
            raise ValueError("tensor dimensions are positive integers or symbols")


@dataclass(frozen=True)
class OpSignature:
    """Identity of one bound operator of a captured step: what it computes, on which tensors, under which layout."""
    semantic_op: str                     # e.g. "linear.cubic4", "attention.paged", "norm.rms", "moe.dispatch"
    phase: BatchPhase
    inputs: tuple[TensorSpec, ...]
    outputs: tuple[TensorSpec, ...]
    accumulator_dtype: str
    layout: str
    shape_items: tuple[tuple[str, int], ...]
    topology_id: str = "single"
    cache_form: str | None = None
    state_form: str | None = None

    def __post_init__(self) -> None:
        if not self.semantic_op or not self.layout or not self.topology_id:
            raise ValueError("operator, layout and topology identities are required")
        if not self.inputs or not self.outputs:
            raise ValueError("an operator has inputs and outputs")
        for kind, ts in (("input", self.inputs), ("output", self.outputs)):
            names = [t.name for t in ts]
            if len(set(names)) != len(names):
                raise ValueError(f"operator {kind} names must be unique")
        keys = [k for k, _ in self.shape_items]
        if keys != sorted(keys) or len(set(keys)) != len(keys) or any(v <= 0 for _, v in self.shape_items):
            raise ValueError("shape items are sorted unique keys with positive values")
        bound = set(keys) | {d for t in self.inputs for d in t.shape if isinstance(d, str)}
        unknown = {d for t in self.outputs for d in t.shape if isinstance(d, str)} - bound
        if unknown:
            raise ValueError("output dimensions must be fixed or bound by an input: " + ", ".join(sorted(unknown)))

    def digest(self) -> str:
        return _digest(asdict(self))


@dataclass(frozen=True)
class EvidenceSeal:
    """A digest that stands for 'this exact thing was qualified': subject kind, subject digest, who sealed it."""
    kind: str
    subject_digest: str
    implementation_digest: str
    device: str
    digest: str = field(default="")

    def __post_init__(self) -> None:
        want = _digest({"kind": self.kind, "subject": self.subject_digest, "impl": self.implementation_digest,
                        "device": self.device})
        if not self.digest:
            object.__setattr__(self, "digest", want)
        elif self.digest != want:
            raise ValueError("evidence seal does not match its contents")


@dataclass(frozen=True)
class ExecutionPlan:
    """What a rank has captured and may replay: the topology, its graph capacities and the operators of a step."""
    topology_id: str
    capacities: tuple[int, ...]
    operators: tuple[OpSignature, ...]
    seals: tuple[EvidenceSeal, ...] = ()

    def __post_init__(self) -> None:
        if list(self.capacities) != sorted(set(self.capacities)) or any(c <= 0 for c in self.capacities):
            raise ValueError("capacities are sorted unique positive row counts")
        if any(o.topology_id != self.topology_id for o in self.operators):
            raise ValueError("every operator of a plan belongs to the plan's topology")

    def digest(self) -> str:
        return _digest({"topology": self.topology_id, "capacities": self.capacities,
                        "operators": [o.digest() for o in self.operators]})

    def seal(self, implementation_digest: str, device: str) -> "ExecutionPlan":
        s = EvidenceSeal("execution-plan", self.digest(), implementation_digest, device)
        return ExecutionPlan(self.topology_id, self.capacities, self.operators, (*self.seals, s))

    def sealed_by(self, implementation_digest: str, device: str) -> bool:
        want = EvidenceSeal("execution-plan", self.digest(), implementation_digest, device).digest
        return any(s.digest == want for s in self.seals)


def decoder_step_operators(cfg, rows: int, tp_size: int = 1, topology_id: str = "single") -> tuple[OpSignature, ...]:
    """Operator signatures of one decode step of a decoder (the shapes the graphs of capacity ``rows`` were captured
    with): what ``cubic qualify`` and the readiness seal identify a captured step by."""
    H, D = cfg.hidden_size, cfg.head_dim
    from ..models.config import kv_heads_of_rank
    hq, hkv = cfg.num_q_heads // tp_size, kv_heads_of_rank(cfg.num_kv_heads, 0, tp_size)[1]
    fmt = f"{cfg.quant.method}{cfg.quant.bits}"
    bf = "bf16"

    def linear(name, n, k):
        return OpSignature(f"linear.{fmt}", BatchPhase.DECODE, (TensorSpec("x", bf, ("m", k)), TensorSpec("w", fmt, (n, k))),
                           (TensorSpec("y", bf, ("m", n)),), "fp32", name, (("k", k), ("m", rows), ("n", n)), topology_id)

    ops = [OpSignature("norm.rms", BatchPhase.DECODE, (TensorSpec("x", bf, ("m", H)),), (TensorSpec("y", bf, ("m", H)),),
                       "fp32", "row", (("h", H), ("m", rows)), topology_id),
           linear("qkv", (hq + 2 * hkv) * D, H),
           OpSignature("attention.paged", BatchPhase.DECODE,
                       (TensorSpec("q", bf, ("m", hq, D)), TensorSpec("kv", "u8", ("pages", hkv, "blob"))),
                       (TensorSpec("o", bf, ("m", hq, D)),), "fp32", "gqa", (("d", D), ("hkv", hkv), ("hq", hq), ("m", rows)),
                       topology_id, cache_form="paged-int-groups32"),
           linear("o", H, hq * D)]
    if cfg.is_moe:
        ops.append(OpSignature("moe.route", BatchPhase.DECODE, (TensorSpec("x", bf, ("m", H)),), (TensorSpec("y", bf, ("m", H)),),
                               "fp32", f"top{cfg.experts_per_token}",
                               (("e", cfg.num_experts), ("h", H), ("i", cfg.moe_intermediate_size), ("m", rows)), topology_id))
    else:
        inter = cfg.intermediate_size // tp_size
        ops += [linear("gate_up", 2 * inter, H), linear("down", H, inter)]
    ops.append(linear("lm_head", cfg.vocab_size // tp_size, H))
    return tuple(ops)
