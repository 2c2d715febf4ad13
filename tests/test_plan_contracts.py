"""Step-level contracts: batch descriptions, state transactions, speculative iterations, operator signatures, seals."""
import pytest

from cubic_serve_b200.contracts.plan import (BatchContract, BatchPhase, EvidenceSeal, ExecutionPlan, OpSignature,
                                             PlanSegment, PrefixPublishPlan, SpeculativeIteration, StateAccess, StateTxn,
                                             TensorSpec, decoder_step_operators, describe_plan)


def test_speculative_iteration_names_what_is_emitted_committed_and_publishable():
    it = SpeculativeIteration(target_state_token_count=37, root_token_id=5, draft_token_ids=(9, 9, 4), accepted_draft_count=2,
                              replacement_token_id=7)
    assert it.verify_token_ids == (5, 9, 9, 4)
    assert it.committed_target_token_ids == (5, 9, 9) and it.committed_target_row_count == 3
    assert it.target_commit_token_count == 40
    assert it.emitted_token_ids == (9, 9, 7) and it.next_root_token_id == 7      # the root was emitted a round earlier
    # only a complete page with a kept recurrent-state checkpoint may be published
    assert it.prefix_checkpoint_boundary(16, (16, 32)) == 32
    assert it.prefix_checkpoint_boundary(16, (16,)) is None
    none = SpeculativeIteration(3, 1, (2,), 0, 8)
    assert none.emitted_token_ids == (8,) and none.committed_target_row_count == 1
    assert none.prefix_checkpoint_boundary(16, (16,)) is None
    with pytest.raises(ValueError):
        SpeculativeIteration(3, 1, (2,), 2, 8)
    with pytest.raises(TypeError):
        SpeculativeIteration(3, 1, [2], 0, 8)


def test_batch_contract_rejects_inconsistent_steps():
    a = PlanSegment("a", BatchPhase.DECODE, True, 33, 1, (4, 5, 6))
    b = PlanSegment("b", BatchPhase.PREFILL, False, 0, 20, (7, 8))
    ok = BatchContract("p1", BatchPhase.MIXED, (a, b), 21, 32, "single", page_copies=((2, 6),))
    assert ok.padding_rows == 11 and len(ok.digest()) == 64
    assert ok.digest() == BatchContract("p1", BatchPhase.MIXED, (a, b), 21, 32, "single", page_copies=((2, 6),)).digest()
    with pytest.raises(ValueError, match="pages"):
        PlanSegment("c", BatchPhase.PREFILL, False, 0, 40, (1, 2))           # 40 tokens need 3 pages
    with pytest.raises(ValueError, match="one token"):
        PlanSegment("c", BatchPhase.DECODE, True, 0, 2, (1,))
    with pytest.raises(ValueError, match="two requests"):
        BatchContract("p", BatchPhase.MIXED, (a, PlanSegment("z", BatchPhase.DECODE, True, 40, 1, (1, 2, 6))), 2, 2, "single")
    with pytest.raises(ValueError, match="logical rows"):
        BatchContract("p", BatchPhase.MIXED, (a, b), 22, 32, "single")
    with pytest.raises(ValueError, match="once per batch"):
        BatchContract("p", BatchPhase.DECODE, (a, a), 2, 2, "single")


def test_state_transactions_are_copy_on_write():
    read = StateAccess("gdn_state", 0, slots=(3,))
    write = StateAccess("gdn_state", 0, slots=(9,))
    txn = StateTxn("t1", "a", 4, 5, (read,), (write,), PrefixPublishPlan(32, 37))
    assert txn.prefix_publish.replay_token_count == 5
    with pytest.raises(ValueError, match="reads and writes"):
        StateTxn("t2", "a", 4, 5, (read,), (StateAccess("gdn_state", 0, slots=(3,)),))
    with pytest.raises(ValueError, match="one revision"):
        StateTxn("t3", "a", 4, 6, (read,), (write,))
    with pytest.raises(ValueError, match="page boundary"):
        PrefixPublishPlan(30, 37)
    seg = PlanSegment("b", BatchPhase.DECODE, True, 33, 1, (4, 5, 6))
    with pytest.raises(ValueError, match="not in the batch"):
        BatchContract("p", BatchPhase.DECODE, (seg,), 1, 1, "single", state_transactions=(txn,))


def test_scheduler_plans_become_contracts():
    from cubic_serve_b200.runtime.engine import LLMEngine
    from cubic_serve_b200.runtime.scheduler import SamplingParams, SchedulerConfig

    class Ex:
        vocab_size = 50

        def copy_pages(self, pairs):
            pass

        def execute(self, segs):
            return [1 for s in segs if s.sample]

    eng = LLMEngine(Ex(), num_pages=32, scheduler_config=SchedulerConfig(max_running_requests=4, max_model_len=128))
    eng.add_request(list(range(20)), SamplingParams(max_tokens=4, ignore_eos=True), "a")
    eng.add_request(list(range(5)), SamplingParams(max_tokens=4, ignore_eos=True), "b")
    plan = eng.scheduler.next_plan()
    c = describe_plan(plan, "step-0", capacity_rows=32)
    assert c.phase is BatchPhase.PREFILL and c.logical_rows == 25 and c.padding_rows == 7
    assert {s.request_id for s in c.segments} == {"a", "b"}


def test_operator_signatures_and_sealed_execution_plans():
    from cubic_serve_b200.models.config import NAMED_CONFIGS
    cfg = NAMED_CONFIGS["dense-8b"]()
    ops = decoder_step_operators(cfg, 256, tp_size=2, topology_id="tp2")
    assert [o.layout for o in ops if o.semantic_op.startswith("linear")] == ["qkv", "o", "gate_up", "down", "lm_head"]
    qkv = ops[1]
    assert dict(qkv.shape_items) == {"k": 4096, "m": 256, "n": (16 + 2 * 4) * 128}
    plan = ExecutionPlan("tp2", (64, 256), ops)
    sealed = plan.seal("impl-digest", "NVIDIA B200")
    assert sealed.sealed_by("impl-digest", "NVIDIA B200") and not sealed.sealed_by("other", "NVIDIA B200")
    assert ExecutionPlan("tp2", (64, 256), decoder_step_operators(cfg, 128, 2, "tp2")).digest() != plan.digest()
    with pytest.raises(ValueError, match="topology"):
        ExecutionPlan("tp4", (64,), ops)
    with pytest.raises(ValueError, match="bound by an input"):
        OpSignature("x", BatchPhase.DECODE, (TensorSpec("a", "bf16", ("m", 4)),), (TensorSpec("b", "bf16", ("q", 4)),), "fp32",
                    "l", (("n", 4),))
    with pytest.raises(ValueError, match="does not match"):
        EvidenceSeal("k", "s", "i", "d", digest="00")
