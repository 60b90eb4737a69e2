"""The kernel tables: a switched-off row is never chosen, every row states its evidence, the
family's shapes resolve to the intended kernels, and refusals keep their reasons
(the invariants MythEclipse/llm tests in apps/engine/src/tactics.rs:454-517)."""
import pytest
import torch

from llm_b200.ops import tactics
from llm_b200.shapes import shape

BF16, F32 = torch.bfloat16, torch.float32


def test_every_row_states_its_evidence_and_ranks_differ():
    for family in ("linear", "attention"):
        rows = tactics.rows(family)
        assert len({r.name for r in rows}) == len(rows)
        assert len({r.rank for r in rows}) == len(rows)          # no tie to break by accident
        for row in rows:
            assert len(row.evidence) > 40, row.name
        assert min(r.rank for r in rows) == 0                      # a row without conditions ends each table


def test_measured_figures_in_the_evidence_are_those_of_the_profiles():
    """A row's evidence quotes measurements; each quoted figure must stand in the summary under
    profiles/ that covers the kernel, so that a table that was not refreshed after a kernel change
    shows up here."""
    import re
    from pathlib import Path
    profiles = Path(__file__).resolve().parent.parent / "profiles"
    evidence = {r.name: r.evidence for family in ("linear", "attention") for r in tactics.rows(family)}
    checks = [("gemm_tc", "gemm_tc_pair__prefill_2048x6144x4096.txt", r"(\d+\.\d) us for 2048 x 6144 x 4096"),
              ("attention_prefill_tc", "attention_prefill_tc__2048_tokens_32x8x128.txt", r"(\d+\.\d) us at 2,048 tokens"),
              ("attention_decode", "attention_decode__batch8_context8192_32x8x128.txt", r"(\d+\.\d) us for 8 sequences")]
    for name, file_name, pattern in checks:
        found = re.search(pattern, evidence[name])
        assert found, (name, evidence[name])
        assert f"{found.group(1)} us" in (profiles / file_name).read_text(), (name, found.group(1), file_name)


def test_switched_off_rows_are_never_chosen():
    args = dict(m=8, n=4096, k=4096, in_dtype=BF16, out_dtype=BF16, lda=4096)
    assert tactics.choose_linear(**args) == "gemm_tc"
    tactics.disable("gemm_tc")
    try:
        assert tactics.choose_linear(**args) == "gemm_skinny"
        assert "not gemm_tc: disabled" in tactics.explain("linear", **args)
        tactics.disable("gemm_skinny")
        assert tactics.choose_linear(**args) == "gemm_simt"
    finally:
        tactics.enable("gemm_tc")
        tactics.enable("gemm_skinny")
    assert tactics.choose_linear(**args) == "gemm_tc"
    assert not tactics.is_disabled("gemm_tc")


@pytest.mark.parametrize("name", ["llama-3.1-8b", "llama-2-7b", "llama-3.2-1b"])
def test_family_shapes_get_the_fast_kernels(name):
    """No shape of the measured configurations falls back silently."""
    from llm_b200.config import config_from_dict
    from llm_b200.engine.model import DecoderModel
    model = DecoderModel(config_from_dict(shape(name, 1)).model_spec())
    for label, family, args in model.kernel_shapes(BF16):
        chosen = tactics._choose(family, **args)[0]
        if family == "linear":
            assert chosen == "gemm_tc", label
        elif label.startswith("decode"):
            assert chosen == "attention_decode", label
        else:
            assert chosen == "attention_prefill_tc", label
    for label, family, args in model.kernel_shapes(F32):           # the 32-bit path: CUDA cores only
        assert tactics._choose(family, **args)[0] in ("gemm_simt", "attention_generic"), label


def test_refusals_name_the_assumption_that_fails():
    text = tactics.explain("attention", decode=True, dtype=BF16, n_heads=32, n_kv_heads=2, head_dim=128,
                           window=0, packed=True)
    assert text.startswith("attention: attention_prefill_tc") and "group of 16 query heads exceeds 8" in text
    text = tactics.explain("attention", decode=False, dtype=BF16, n_heads=4, n_kv_heads=4, head_dim=80,
                           window=0, packed=True)
    assert text.startswith("attention: attention_generic") and "head_dim 80" in text
    text = tactics.explain("attention", decode=True, dtype=BF16, n_heads=4, n_kv_heads=2, head_dim=64,
                           window=100, packed=True)
    assert text.startswith("attention: attention_generic") and "no window" in text
    text = tactics.explain("linear", m=2048, n=4096, k=4100, in_dtype=BF16, out_dtype=BF16, lda=4100)
    assert text.startswith("linear: gemm_simt") and "multiple of 8" in text and "exceed 64" in text


def test_a_head_size_no_kernel_takes_is_refused_by_name():
    """Above 256 no attention kernel runs: the choice fails and says so, for the model as a whole
    too (an engine computes the model's kernel plan when it is built)."""
    from llm_b200.config import config_from_dict
    from llm_b200.engine.model import DecoderModel
    from llm_b200.errors import LlmError
    with pytest.raises(LlmError, match="head_dim 272 exceeds 256"):
        tactics.choose_attention(True, BF16, 4, 2, 272, 0)
    raw = shape("llama-3.2-1b", 1)
    raw["head_dim"] = 272
    model = DecoderModel(config_from_dict(raw).model_spec())
    with pytest.raises(LlmError, match="no kernel accepts the shape"):
        model.plan_identity(BF16)
    assert tactics.choose_attention(False, F32, 4, 2, 256, 0) == "attention_generic"
