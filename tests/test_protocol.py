"""Every executor that ships satisfies the engine's executor protocol; incomplete ones are named."""
import numpy as np
import pytest

from cubic_serve_b200.models import protocol as P


def test_shipped_cpu_executors_conform():
    from cubic_serve_b200.executor.eager_executor import EagerPagedExecutor
    from cubic_serve_b200.models import eager_family as EF
    from cubic_serve_b200.models import qwen4_exp as Q
    from cubic_serve_b200.models.config import ModelConfig
    from cubic_serve_b200.models.reference import random_dense_weights
    cfg = ModelConfig()
    paged = EagerPagedExecutor(cfg, random_dense_weights(cfg, 0), 8)
    caps = P.check_executor(paged)
    assert isinstance(paged, P.StepExecutor) and caps.features and not caps.request_state and not caps.overlapped
    fam = EF.EagerFamilyExecutor(cfg, EF.random_family_weights(cfg, 0))
    assert P.check_executor(fam).request_state
    q4 = Q.Qwen4ExpEagerExecutor(Q.tiny_config(), Q.random_qwen4_exp_weights(Q.tiny_config(), 0))
    caps4 = P.check_executor(q4)                                  # it also runs draft-head rounds
    assert caps4.request_state and caps4.features and caps4.speculative and isinstance(q4, P.SpeculativeExecutor)


def test_native_executor_classes_state_their_capabilities():
    from cubic_serve_b200.executor.gpu_executor import GpuExecutor
    from cubic_serve_b200.executor.spec_executor import NgramSpeculativeGpuExecutor, SpeculativeGpuExecutor
    for cls in (GpuExecutor, SpeculativeGpuExecutor, NgramSpeculativeGpuExecutor):
        assert all(callable(getattr(cls, n, None)) for n in ("execute", "copy_pages", "launch", "collect"))
    assert callable(SpeculativeGpuExecutor.execute_speculative) and callable(GpuExecutor.copy_state)


def test_incomplete_executors_are_named():
    class NoCopy:
        def execute(self, segs):
            return np.zeros(0, np.int32)

    class HalfOverlap(NoCopy):
        def copy_pages(self, pairs):
            pass

        def launch(self, segs, feedback_rows=0):
            pass

    class Rows(NoCopy):
        state_checkpoint_rows = (4, 5)

        def copy_pages(self, pairs):
            pass
    with pytest.raises(TypeError, match="copy_pages"):
        P.check_executor(NoCopy())
    with pytest.raises(TypeError, match="counterpart"):
        P.check_executor(HalfOverlap())
    with pytest.raises(TypeError, match="snapshot rows"):
        P.check_executor(Rows())
    assert not isinstance(NoCopy(), P.StepExecutor)
