"""The eager PyTorch functions of triton_kernels_b200.functional against outputs of the
reference's own functional package (triton_kernels/functional/normalization.py:6-25,
triton_kernels/functional/positional_embedding.py:5-10) stored in tests/golden/.  CPU only."""
import cases
import torch

from triton_kernels_b200 import functional as F


def _same_inputs(case, golden_case):
    for name, fp in golden_case["fp"].items():
        assert cases.fingerprint(case[name]) == fp, f"regenerated input {name!r} differs from the golden run's"


def test_rms_norm_torch_matches_reference(golden):
    c = cases.case_rms_norm()
    _same_inputs(c, golden["rms_norm"])
    for fn in (F.rms_norm_torch, F.rms_norm_torch_compile):
        torch.testing.assert_close(fn(c["x"], c["scale"]), golden["rms_norm"]["y"], atol=1e-6, rtol=1e-6)


def test_layer_norm_modulation_torch_matches_reference(golden):
    c = cases.case_layer_norm_modulation()
    _same_inputs(c, golden["layer_norm_modulation"])
    for fn in (F.layer_norm_modulation_torch, F.layer_norm_modulation_torch_compile):
        torch.testing.assert_close(fn(c["x"], c["scale"], c["shift"]), golden["layer_norm_modulation"]["y"],
                                   atol=2e-5, rtol=1e-5)


def test_apply_rope_torch_matches_reference(golden):
    c = cases.case_rope_random_table()
    _same_inputs(c, golden["rope_random_table"])
    for fn in (F.apply_rope_torch, F.apply_rope_torch_compile):
        q, k = fn(c["q"], c["k"], c["pe"])
        torch.testing.assert_close(q, golden["rope_random_table"]["q"], atol=1e-6, rtol=1e-6)
        torch.testing.assert_close(k, golden["rope_random_table"]["k"], atol=1e-6, rtol=1e-6)


def test_functional_keeps_input_dtype():
    x = torch.randn(2, 5, 128).to(torch.bfloat16)
    assert F.rms_norm_torch(x, torch.ones(128, dtype=torch.bfloat16)).dtype == torch.bfloat16
    q, k = F.apply_rope_torch(x[:, None], x[:, None], torch.randn(1, 1, 5, 64, 2, 2))
    assert q.dtype == torch.bfloat16 and k.shape == (2, 1, 5, 128)
