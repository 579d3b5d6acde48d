"""The plain implementation against the reference project's own fixture.

The fixture's logits were computed by the reference's authors with an
independent implementation (float32, eager attention, no cache); the
reference's own bar for its CPU runner is 2e-6 absolute (test/qwen.test.ts:35).
"""
import json

import numpy as np

import plain_qwen2 as plain


def test_fixture_logits_within_reference_tolerance(fixture_dir):
    cfg, w = plain.read_model_folder(fixture_dir)
    record = json.loads((fixture_dir / "reference.json").read_text())
    worst = 0.0
    for case in record["cases"]:
        history = list(case["tokens"])
        for step, name in enumerate(case["logits"]):
            want = np.fromfile(fixture_dir / name, dtype="<f4")
            got = plain.logits(cfg, w, history)[-1]
            worst = max(worst, float(np.abs(got - want).max()))
            assert int(np.argmax(got)) == case["output"][step]
            history.append(case["output"][step])
    assert worst < 2e-6, worst


def test_golden_copy_is_the_reference_fixture():
    """tests/golden/qwen-tiny is a byte-identical copy of the reference's data files."""
    import conftest
    import pytest
    checkout = conftest.reference_checkout_fixture_dir()
    if checkout is None:
        pytest.skip("no checkout of the reference project at hand")
    names = sorted(p.name for p in conftest.GOLDEN_FIXTURE.iterdir())
    assert "model.safetensors" in names and len([n for n in names if n.endswith(".f32")]) == 8
    for name in names:
        assert (checkout / name).read_bytes() == (conftest.GOLDEN_FIXTURE / name).read_bytes(), name


def test_fixture_greedy_outputs(fixture_dir):
    cfg, w = plain.read_model_folder(fixture_dir)
    record = json.loads((fixture_dir / "reference.json").read_text())
    for case in record["cases"]:
        assert plain.greedy(cfg, w, case["tokens"], len(case["output"])) == case["output"]


def test_parts_shapes_and_simple_values():
    x = np.array([[3.0, 4.0]], dtype=np.float32)
    out = plain.rms_norm(x, np.array([1.0, 2.0], dtype=np.float32), 0.0)
    scale = 1.0 / np.sqrt(12.5)
    np.testing.assert_allclose(out, [[3 * scale, 8 * scale]], rtol=1e-6)
    # rotation at position 0 is the identity; at any position it keeps the norm
    v = np.arange(8, dtype=np.float32).reshape(1, 8)
    np.testing.assert_array_equal(plain.rope_half_split(v, [0], 4, 10000.0), v)
    r = plain.rope_half_split(v, [5], 4, 10000.0)
    np.testing.assert_allclose(np.linalg.norm(r), np.linalg.norm(v), rtol=1e-6)
    # pairs are (d, d + half): rotating a unit vector on axis 0 of a head moves weight to axis half
    e = np.zeros((1, 4), dtype=np.float32); e[0, 0] = 1
    r = plain.rope_half_split(e, [1], 4, 10000.0)
    np.testing.assert_allclose(r[0], [np.cos(1.0), 0, np.sin(1.0), 0], atol=1e-7)
    g = plain.swiglu(np.array([0.0, 1.0], np.float32), np.array([5.0, 2.0], np.float32))
    np.testing.assert_allclose(g, [0.0, 2.0 / (1 + np.exp(-1.0))], rtol=1e-6)


def test_attention_single_position_returns_value():
    q = np.ones((1, 4), np.float32)
    k = np.ones((1, 2), np.float32)
    v = np.array([[7.0, 9.0]], np.float32)
    out = plain.causal_gqa_attention(q, k, v, heads=2, kv_heads=1, head_dim=2)
    np.testing.assert_array_equal(out, [[7, 9, 7, 9]])
