"""The scratch planner: buffers that are live together never share bytes, buffers whose
lifetimes are disjoint do share, everything is aligned, the identity follows the layout
(the invariants MythEclipse/llm tests on its planner, apps/engine/src/workspace.rs:344-438)."""
import random

import pytest
import torch

from tiny import make_folder

from llm_b200.engine.workspace import ALIGNMENT, BufferRequest, Workspace, plan


def req(name, n, first, last, dtype=torch.bfloat16):
    return BufferRequest(name, (n,), dtype, first, last)


def test_disjoint_lifetimes_share_and_live_ones_do_not():
    p = plan([req("a", 1000, 0, 1), req("b", 1000, 1, 2), req("c", 1000, 2, 3), req("d", 300, 3, 3)])
    p.check()
    at = {n: pl.offset for n, pl in p.placements.items()}
    assert at["a"] == 0 and at["b"] != at["a"]            # b is written while a is still read
    assert at["c"] == at["a"]                             # a is dead when c is born
    assert p.total < 4 * 2000 and p.total % ALIGNMENT == 0
    assert all(o % ALIGNMENT == 0 for o in at.values())


def test_random_requests_never_overlap_while_live():
    rng = random.Random(1)
    for trial in range(50):
        requests = []
        for i in range(rng.randint(1, 25)):
            first = rng.randint(0, 9)
            requests.append(BufferRequest(f"b{i}", (rng.randint(1, 4000),),
                                          rng.choice([torch.float32, torch.bfloat16, torch.int32]),
                                          first, first + rng.randint(0, 4)))
        p = plan(requests)
        p.check()
        assert p.total <= sum(-(-r.nbytes // ALIGNMENT) * ALIGNMENT for r in requests)


def test_identity_follows_the_layout_and_bad_requests_are_refused():
    a = plan([req("x", 100, 0, 1), req("y", 100, 1, 2)])
    b = plan([req("y", 100, 1, 2), req("x", 100, 0, 1)])
    c = plan([req("x", 100, 0, 2), req("y", 100, 1, 2)])
    assert a.identity() == b.identity() != c.identity()
    with pytest.raises(ValueError):
        plan([req("x", 1, 0, 1), req("x", 2, 0, 1)])
    with pytest.raises(ValueError):
        plan([req("x", 1, 3, 2)])


def test_a_model_declares_its_scratch_and_gets_views(tmp_path):
    from llm_b200.engine import load_model
    model = load_model(make_folder(tmp_path, "B", torch.bfloat16), torch.bfloat16, "cpu")
    requests = model.scratch_requests(10)
    names = {r.name for r in requests}
    assert {"h_mixer", "mixer.qkv", "mixer.mixed", "h_ffn", "ffn.act"} <= names
    shapes = {r.name: r.shape for r in requests}
    assert shapes["mixer.qkv"] == (10, (3 + 2) * 32) and shapes["ffn.act"] == (10, 256)
    workspace = Workspace("cpu", model.scratch_requests)
    views = workspace.for_tokens(10)
    views.plan.check()
    views.prefix = "mixer."
    qkv = views.get("qkv")
    assert qkv.shape == (10, 160) and qkv.dtype == torch.bfloat16 and views.get("nothing") is None
    first_arena = workspace.arena
    big = workspace.for_tokens(500)                  # a larger step: a new arena, the old one is kept
    assert workspace.arena.numel() >= big.plan.total and workspace._retired == [first_arena]
    assert workspace.for_tokens(10).arena is workspace.arena
    # the attention output reuses the bytes of the normed input: their lifetimes do not meet
    assert views.plan.total < sum(r.nbytes for r in requests)


def test_kernel_plan_and_build_identities(tmp_path):
    """The kernel plan's identity changes exactly when a selection changes; the build identity
    is one hash over the native sources, the flags and the compiler."""
    from llm_b200.config import config_from_dict
    from llm_b200.engine.model import DecoderModel
    from llm_b200.ops import tactics
    from llm_b200.ops.build import build_identity
    from tiny import TINY_F
    model = DecoderModel(config_from_dict(dict(TINY_F)).model_spec())
    shapes = model.kernel_shapes(torch.bfloat16)
    labels = [label for label, _, _ in shapes]
    assert "prefill attention" in labels and "decode attention" in labels
    assert any(label.startswith("head product") for label in labels)
    before = model.plan_identity(torch.bfloat16)
    assert before == model.plan_identity(torch.bfloat16) and len(before) == 16
    tactics.disable("attention_prefill_tc")
    try:
        assert model.plan_identity(torch.bfloat16) != before
    finally:
        tactics.enable("attention_prefill_tc")
    assert model.plan_identity(torch.bfloat16) == before
    assert model.plan_identity(torch.float32) != before         # the 32-bit path picks other kernels
    assert build_identity() == build_identity() and len(build_identity()) == 16
