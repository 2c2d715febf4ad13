import torch

from cubic_serve_b200.guardrail.compare import DifferenceClass, compare_tensors, poisoned_padding_preserved, reduction_bound


def test_compare_classes():
    o = torch.randn(8, 16)
    assert compare_tensors(o.clone(), o, 1e-3).klass is DifferenceClass.EXACT
    b = reduction_bound(o, torch.bfloat16, 4096)
    near = o.to(torch.bfloat16).float()
    v = compare_tensors(near, o, b)
    assert v.klass is DifferenceClass.ROUNDING and v.ok and v.rel_l2 < b
    far = o.clone(); far[3, 5] += 10
    v = compare_tensors(far, o, b)
    assert v.klass is DifferenceClass.MISMATCH and v.worst_index == (3, 5) and not v.ok
    nan = o.clone(); nan[1, 2] = float("nan")
    assert compare_tensors(nan, o, b).klass is DifferenceClass.MISMATCH
    assert compare_tensors(o[:4], o, b).klass is DifferenceClass.MISMATCH
    assert poisoned_padding_preserved(o, o.clone()) and not poisoned_padding_preserved(o, far)
