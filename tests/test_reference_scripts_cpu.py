"""The reference's own test scripts, run unmodified against this framework through the ``moe_arch`` import shim.

The scripts (print-driven, each with a ``main``) live in the reference's source tree, not in its installed package;
they are looked for in ``$KMOE_REFERENCE_SRC`` or in a directory ``reference`` beside this repository, and the
tests are skipped where there is none.  Each script is started in a child process that imports this repository's
``moe_arch`` first, so that the script's own ``sys.path`` entry for its tree no longer decides what ``moe_arch``
is.  A script passes when it exits 0, prints its check marks and no failure mark.

Not run: ``test_3b_config.py`` (builds a 14-billion-parameter model on the host), ``tests/test_phase2_moe.py`` and
``tests/test_phase3_complete.py`` (they use an older interface and stop at the same line on the reference itself:
``layer.ffn.router`` of a dense layer, three results from the four-result MoD router), and the scripts that need
a data set from the hub.
"""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.environ.get("KMOE_REFERENCE_SRC") or os.path.join(os.path.dirname(ROOT), "reference")
pytestmark = pytest.mark.skipif(not os.path.isfile(os.path.join(SRC, "test_gradient_flow.py")),
                                reason="the reference's source tree (with its test scripts) is not available")

RUNNER = (
    "import sys, runpy\n"
    "sys.path.insert(0, {root!r})\n"
    "import moe_arch\n"                                   # the shim is in sys.modules before the script runs
    "assert moe_arch.__file__.startswith({root!r}), moe_arch.__file__\n"
    "import random, torch\n"                              # the scripts draw unseeded inputs and compare
    "random.seed(0); torch.manual_seed(0)\n"             # against thresholds: make every run the same run
    "sys.argv = [{script!r}]\n"
    "runpy.run_path({script!r}, run_name='__main__')\n")


@pytest.mark.parametrize("script,min_checks", [
    ("test_attention_mask_fix.py", 2),           # padding positions do not count in the loss when a mask is given
    ("test_gradient_flow.py", 20),               # every parameter group receives gradient, with and without MoD
    ("test_muon_conv_fix.py", 5),                # Muon on conv kernels (>= 3-D tensors are flattened)
    ("test_muon_with_model.py", 6),              # hybrid optimizer on the whole model, a few steps
    ("verify_routing_mamba_fix.py", 8),          # RoutingMamba where a layer is both Mamba and MoE
    ("tests/test_phase4_training.py", 20),       # tokenizer, data, schedule, Muon, trainer, checkpoint, pipeline
    # shapes, loss, gradients, generation and an 8-layer cut of the 5B preset: two minutes on a CPU, so only with
    # KMOE_SLOW_TESTS=1 (the script reads ``count_parameters()["lm_head"]``, which the reference itself lacks)
    pytest.param("tests/test_phase1_mvp.py", 10,
                 marks=pytest.mark.skipif(os.environ.get("KMOE_SLOW_TESTS") != "1", reason="slow: KMOE_SLOW_TESTS=1")),
])
def test_reference_script_passes_on_this_framework(script, min_checks, tmp_path):
    path = os.path.join(SRC, script)
    env = dict(os.environ, KMOE_OFFLINE="1", HF_HUB_OFFLINE="1", CUDA_VISIBLE_DEVICES="", MOE_DISABLE_COMPILE="1")
    r = subprocess.run([sys.executable, "-c", RUNNER.format(root=ROOT, script=path)], cwd=str(tmp_path), env=env,
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    tail = r.stdout[-3000:]
    assert r.returncode == 0, tail
    assert r.stdout.count("✓") >= min_checks, tail
    assert "✗" not in r.stdout and "Traceback" not in r.stdout, tail


def test_layer_configuration_equals_the_reference_s_committed_sample(capsys):
    """The reference ships a cluster analysis and the per-layer configuration its generator made from it
    (``sparse_distillation_output/``): this framework's generator gives the same layers and the same totals."""
    import json
    from experiments.sparse_distillation.generate_config import compute_layer_config
    d = os.path.join(SRC, "sparse_distillation_output")
    if not os.path.isfile(os.path.join(d, "layer_config.json")):
        pytest.skip("no sample output in the reference tree")
    analysis = json.load(open(os.path.join(d, "cluster_analysis.json")))
    gold = json.load(open(os.path.join(d, "layer_config.json")))
    ours = compute_layer_config(analysis, gold["target_expansion_ratio"], gold["target_active_ratio"], gold["min_experts"])
    capsys.readouterr()
    assert set(ours["layers"]) == set(gold["layers"]) and len(gold["layers"]) > 0
    for k, g in gold["layers"].items():
        assert {x: ours["layers"][k][x] for x in ("n_experts", "d_ff_expert", "top_k")} == \
               {x: g[x] for x in ("n_experts", "d_ff_expert", "top_k")}, k
    for k, v in gold["stats"].items():
        assert ours["stats"][k] == pytest.approx(v), k


MAKE_REFERENCE_CHECKPOINT = r"""
import sys, torch
sys.path.insert(0, {src!r})
from Experiments.sparse_distillation import distill as ref_distill      # imported before this repository is on
import moe_arch                                                         # the path: the reference's own code
from Experiments.sparse_distillation.distill import DistillationConfig, SparseDistillationTrainer
assert ref_distill.__file__.startswith({src!r}) and moe_arch.__file__.startswith({src!r})
sys.path.insert(1, {root!r})
from experiments.sparse_distillation.example_usage import ToyLM          # only the toy teacher comes from this repo
torch.manual_seed(0)
m = ToyLM().eval()
cfg = DistillationConfig(n_experts=4, moe_top_k=2, moe_routing={routing!r}, d_ff_expert=64, data_free=True,
                         data_free_steps=3, data_free_batch_size=2, data_free_seq_len=16, use_compile=False,
                         supervised_routing=False, log_interval=1000, router_mlp={mlp!r})
tr = SparseDistillationTrainer(dense_model=m, config=cfg, device="cpu")
tr.distill()
tr.save({out!r} + "/distilled.pt")
torch.save(m.state_dict(), {out!r} + "/teacher.pt")
x = torch.randn(2, 16, 64)
with torch.no_grad():
    torch.save({{"x": x, "y0": tr.moe_layers["0"](x), "y1": tr.moe_layers["1"](x)}}, {out!r} + "/io.pt")
"""


@pytest.mark.parametrize("routing,mlp", [("token_choice", False), ("expert_choice", False), ("token_choice", True)])
def test_distillation_checkpoint_of_the_reference_loads_and_computes_the_same(routing, mlp, tmp_path):
    """A checkpoint written by the reference's own ``SparseDistillationTrainer`` (run in a child process on its
    code) is read by ``convert_to_sparse`` here, and the converted layers map the same input to the same output."""
    import torch
    from experiments.sparse_distillation.convert import convert_to_sparse
    from experiments.sparse_distillation.example_usage import ToyLM
    code = MAKE_REFERENCE_CHECKPOINT.format(src=SRC, root=ROOT, out=str(tmp_path), routing=routing, mlp=mlp)
    env = dict(os.environ, MOE_DISABLE_COMPILE="1", CUDA_VISIBLE_DEVICES="", HF_HUB_OFFLINE="1")
    r = subprocess.run([sys.executable, "-c", code], cwd=str(tmp_path), env=env, stdout=subprocess.PIPE,
                       stderr=subprocess.STDOUT, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:]
    m = ToyLM().eval()
    m.load_state_dict(torch.load(tmp_path / "teacher.pt"))
    wrapper = convert_to_sparse(dense_model=m, distillation_checkpoint=str(tmp_path / "distilled.pt"), device="cpu")
    io = torch.load(tmp_path / "io.pt")
    layers = wrapper.moe_layers
    assert layers["0"].routing == routing and layers["0"].n_experts == 4 and layers["0"].d_ff == 64
    with torch.no_grad():
        for k in ("0", "1"):
            assert torch.allclose(layers[k](io["x"]), io["y" + k], atol=1e-6), (routing, mlp, k)
