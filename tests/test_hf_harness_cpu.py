"""Host-side pieces of the generation harness (b200k/hf_harness.py) against the reference's own
benchmarks/utils.py, imported from a checkout when one is at hand (REFERENCE_ROOT, or a `reference`
directory beside the repo): the size formulas, the log text and the behaviour of the timing hooks."""
import os
import types

import pytest
import torch

from b200k import hf_harness

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def reference_utils():
    root = os.environ.get("REFERENCE_ROOT") or os.path.join(os.path.dirname(ROOT), "reference")
    if not os.path.exists(os.path.join(root, "benchmarks", "utils.py")):
        pytest.skip("no reference checkout at hand")
    return hf_harness.load_reference_utils(root)


CONFIGS = [types.SimpleNamespace(hidden_size=h, num_hidden_layers=n, vocab_size=v)
           for (h, n, v) in ((4096, 32, 32000), (1024, 2, 1000), (8192, 80, 128256))]


def test_size_formulas_and_log_text_match_the_reference(reference_utils):
    for cfg in CONFIGS:
        assert hf_harness.model_bytes(cfg) == reference_utils.model_bytes(cfg)
        assert hf_harness.cache_bytes(cfg, 7, 544) == reference_utils.cache_bytes(cfg, 7, 544)
    args = (13.5e9, 2.1e9, 30.25e9, 0.12345, 33177.6, 1.98765, 249.49, 2.1111, 242.5)
    assert hf_harness.write_gen_benchmark_log(*args) == reference_utils.write_gen_benchmark_log(*args)


def test_llama2_7b_model_bytes_value():
    cfg = types.SimpleNamespace(hidden_size=4096, num_hidden_layers=32, vocab_size=32000)
    # 2 * (32 * (12 h^2 + 11 h) + 32000 * (h + 1)), h = 4096
    assert hf_harness.model_bytes(cfg) == 2 * (32 * (12 * 4096 ** 2 + 11 * 4096) + 32000 * 4097)


class _Tiny(torch.nn.Module):
    def forward(self, x):
        return x + 1


def _drive(utils, monkeypatch):
    """Two forwards in the prefill stage protocol of hf-gen.py, then removal; returns what was seen."""
    monkeypatch.setattr(torch.cuda, "synchronize", lambda *a, **k: None)
    m = _Tiny()
    utils.add_model_hooks(m)
    utils.add_model_hooks(m)          # idempotent: no second pair of hooks
    seen = []
    m.stage = "prefill"
    m(torch.zeros(1))
    seen.append((m.stage, hasattr(m, "__duration__") and m.__duration__ >= 0))
    first = m.__duration__
    m(torch.zeros(1))                 # decode stage: untouched
    seen.append((m.stage, m.__duration__ == first))
    utils.remove_model_hooks(m)
    seen.append((hasattr(m, "stage"), hasattr(m, "__duration__"), len(m._forward_hooks), len(m._forward_pre_hooks)))
    return seen


def test_timing_hooks_behave_like_the_reference(reference_utils, monkeypatch):
    mine = _drive(hf_harness, monkeypatch)
    theirs = _drive(reference_utils, monkeypatch)
    assert mine[:2] == theirs[:2] == [("decode", True), ("decode", True)]
    # the reference leaves one pre-hook behind when asked twice (its first guard tests a different
    # attribute name than it sets, benchmarks/utils.py:91-93); this module removes everything it added
    assert mine[2] == (False, False, 0, 0) and theirs[2][:3] == (False, False, 0)


def test_harness_utils_prefers_the_reference_checkout(reference_utils, monkeypatch):
    root = os.path.dirname(os.path.dirname(reference_utils.__file__))
    monkeypatch.setenv("REFERENCE_ROOT", root)
    assert hf_harness.harness_utils().__file__ == reference_utils.__file__
    monkeypatch.setenv("REFERENCE_ROOT", "")
    assert hf_harness.harness_utils() is hf_harness


def test_fine_linear_layout_and_routing_count():
    lin = torch.nn.Linear(24, 40, bias=False)
    fl = hf_harness.FineLinear(lin)
    assert fl.weight_kn.shape == (24, 40) and torch.equal(fl.weight_kn, lin.weight.t())
    with pytest.raises(RuntimeError):
        hf_harness.FineLinear(torch.nn.Linear(4, 4, bias=True))
    net = torch.nn.Sequential(torch.nn.Linear(8, 8, bias=False), torch.nn.ReLU(), torch.nn.Linear(8, 8, bias=True))
    assert hf_harness.route_linears_through_gemm_unified(net) == 1
    assert isinstance(net[0], hf_harness.FineLinear) and isinstance(net[2], torch.nn.Linear)
