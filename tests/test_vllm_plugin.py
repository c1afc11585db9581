"""This package as a hardware plugin of the installed upstream vLLM.

``vllm.LLM`` is the entry point; vLLM's engine core, scheduler and block pool are untouched; the
platform plugin makes vLLM's executor construct this package's ``WorkerBase`` subclass, which runs
this package's model, paged KV cache and kernels on the block ids vLLM hands out.  The checks: the
platform and the worker are the plugin's, greedy tokens equal those of this package's own engine
on the same random-init weights (synchronous stepping, asynchronous scheduling, and with
preemption + resume under a KV cache that is too small), and on a GPU the native library is mapped
and its kernels were launched.

Counterpart in the reference: the five entry points of setup.py:518-529 and
``NPUWorker(WorkerBase)`` (vllm_ascend/worker/worker.py:98)."""
import json
import os
import subprocess
import sys

import pytest
import torch

vllm = pytest.importorskip("vllm")

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WORKER = os.path.join(ROOT, "tests", "vllm_plugin_worker.py")

TINY = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=1024, hidden_size=256,
            intermediate_size=512, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
            head_dim=64, rms_norm_eps=1e-6, rope_theta=1e6, max_position_embeddings=4096,
            tie_word_embeddings=False, hidden_act="silu", attention_bias=False)


def _model_dir(tmp_path, dtype, **over):
    d = tmp_path / "tiny-qwen3"
    d.mkdir(exist_ok=True)
    (d / "config.json").write_text(json.dumps(dict(TINY, torch_dtype=dtype, **over)))
    return str(d)


def _run(site_dir, model_dir, dtype, mode, timeout=900):
    env = dict(os.environ)
    env.pop("VLLM_PLUGINS", None)
    res = subprocess.run([sys.executable, WORKER, site_dir, model_dir, dtype, mode], env=env, cwd=str(os.path.dirname(model_dir)),
                         capture_output=True, text=True, timeout=timeout)
    assert res.returncode == 0, (res.stdout[-2000:], res.stderr[-4000:])
    line = [l for l in res.stdout.splitlines() if l.startswith("RESULT ")][-1]
    return json.loads(line[7:])


def _check_common(r):
    assert r["platform"] == "B200Platform"
    assert r["worker"] == "B200VllmWorker"
    assert all(len(t) > 0 for t in r["got"])


def test_vllm_prompt_embedding_requests_on_the_plugin_cpu(tmp_path):
    r = _run("", _model_dir(tmp_path, "float32"), "float32", "embeds")
    _check_common(r)
    assert r["got"] == r["want"]


def test_vllm_structured_outputs_reach_the_plugin_sampler_cpu(tmp_path):
    """vLLM compiles the grammar and hands the worker one token bitmask per step; the worker runs the
    forward pass, applies the bitmask to the rows of the constrained requests and samples."""
    r = _run("", _model_dir(tmp_path, "float32"), "float32", "structured")
    _check_common(r)
    assert r["texts"][0] in r["choices"] and r["texts"][2] in r["choices"]
    assert len(r["got"][1]) == 6 and len(r["got"][3]) == 6
    assert [r["got"][1], r["got"][3]] == r["free_alone"]


@pytest.mark.parametrize("mode", ["sync", "async"])
def test_vllm_llm_runs_on_the_plugin_and_matches_the_own_engine_cpu(tmp_path, mode):
    r = _run("", _model_dir(tmp_path, "float32"), "float32", mode)
    _check_common(r)
    assert r["async"] == (mode == "async")
    assert r["got"] == r["want"]


def test_vllm_preemption_and_resume_on_the_plugin_cpu(tmp_path):
    r = _run("", _model_dir(tmp_path, "float32"), "float32", "preempt")
    _check_common(r)
    assert r["stats"]["preempted"] > 0 and r["stats"]["resumed"] > 0
    assert r["got"] == r["want"]


def test_entry_points_declared_in_pyproject():
    text = open(os.path.join(ROOT, "pyproject.toml")).read()
    assert '[project.entry-points."vllm.platform_plugins"]' in text
    assert '[project.entry-points."vllm.general_plugins"]' in text
    for hook in ("register", "register_connector", "register_model_loader", "register_service_profiling",
                 "register_model"):
        assert f"vllm_ascend_b200:{hook}" in text
    import vllm_ascend_b200
    assert vllm_ascend_b200.register() == "vllm_ascend_b200.platform.B200Platform"


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["sync", "async", "preempt"])
def test_vllm_llm_runs_on_the_plugin_gpu(tmp_path, mode):
    """Offline editable install into a private prefix (``pip install -e . --no-build-isolation
    --no-deps --no-index``): vLLM discovers the plugin from the installed distribution's entry points."""
    prefix = tmp_path / "prefix"
    res = subprocess.run([sys.executable, "-m", "pip", "install", "-e", ROOT, "--no-build-isolation", "--no-deps",
                          "--no-index", "--prefix", str(prefix), "-q"], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-3000:]
    site_dir = str(prefix / "lib" / f"python{sys.version_info.major}.{sys.version_info.minor}" / "site-packages")
    assert os.path.isdir(site_dir)
    r = _run(site_dir, _model_dir(tmp_path, "bfloat16", head_dim=128, num_attention_heads=8, hidden_size=512,
                                  intermediate_size=1024), "bfloat16", mode)
    _check_common(r)
    assert r["installed"] and r["device"].startswith("cuda")
    assert r["native_mapped"], "the native library was not loaded under vLLM"
    assert r["launches"] > 0, "no kernel of this package ran under vLLM"
    if mode == "preempt":
        assert r["stats"]["preempted"] > 0 and r["stats"]["resumed"] > 0
    agree = sum(a == b for x, y in zip(r["got"], r["want"]) for a, b in zip(x, y)) / sum(len(x) for x in r["want"])
    # same kernels, same weights; batch composition may differ between the two schedulers, which
    # moves bf16 near-ties only
    assert agree > 0.9, (agree, r["got"], r["want"])
