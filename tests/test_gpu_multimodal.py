"""Multimodal kernels against their PyTorch definitions; the vision-language model on the engine."""
import numpy as np
import pytest
import torch

from vllm_ascend_b200 import _native, ops
from vllm_ascend_b200.ops import mm_encoder as enc
from vllm_ascend_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("D,sections,interleaved", [(128, [16, 24, 24], False), (128, [24, 20, 20], True),
                                                   (64, [8, 12, 12], False)])
def test_mrope_kernel(D, sections, interleaved):
    g = torch.Generator().manual_seed(0)
    T, Hq, Hkv = 67, 8, 2
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, generator=g).bfloat16()
    pos = torch.randint(0, 500, (3, 80), generator=g)
    cs = ref.build_cos_sin_cache(D, 512, 1e6, None, "cpu")
    axis = ref.mrope_axis_table(sections, interleaved)
    qn, kn = torch.rand(D, generator=g).bfloat16() + 0.5, torch.rand(D, generator=g).bfloat16() + 0.5
    kc = torch.zeros(4, 32, Hkv, D).bfloat16()
    vc = torch.zeros_like(kc)
    slots = torch.randperm(128, generator=g)[:T]
    want = qkv.clone().float()
    kc_ref, vc_ref = kc.clone().float(), vc.clone().float()
    ref.qknorm_rope_kvwrite(want, pos, cs, D, qn.float(), kn.float(), 1e-6, kc_ref, vc_ref, slots, Hq, Hkv, D,
                            mrope_axis=axis)
    q_dev, kc_dev, vc_dev = qkv.to(DEV), kc.to(DEV), vc.to(DEV)
    ops.qknorm_rope_kvwrite(q_dev, pos.to(DEV), cs.to(DEV), D, qn.to(DEV), kn.to(DEV), 1e-6, kc_dev, vc_dev,
                            slots.to(DEV), Hq, Hkv, D, mrope_axis=axis.to(DEV))
    torch.cuda.synchronize()
    _native.check_status(torch.device(DEV))
    assert (q_dev.float().cpu() - want).abs().max() < 6e-2
    assert (kc_dev.float().cpu() - kc_ref).abs().max() < 6e-2
    assert (vc_dev.float().cpu() - vc_ref).abs().max() < 1e-2


def test_rope_table_kernel():
    g = torch.Generator().manual_seed(1)
    N, H, D = 300, 6, 80
    x = torch.randn(N, 3 * H, D, generator=g).bfloat16()
    ang = torch.rand(N, D // 2, generator=g) * 6
    cos, sin = ang.cos(), ang.sin()
    want = enc.rope_table_ref(x[:, :2 * H].float(), cos, sin)
    xd = x.to(DEV)
    enc.rope_table_(xd[:, :2 * H], cos.to(DEV), sin.to(DEV))
    torch.cuda.synchronize()
    assert (xd[:, :2 * H].float().cpu() - want).abs().max() < 3e-2
    assert torch.equal(xd[:, 2 * H:].cpu(), x[:, 2 * H:])


@pytest.mark.parametrize("D", [80, 64, 128])
def test_encoder_attention_kernel(D):
    g = torch.Generator().manual_seed(2)
    lens = [64, 300, 1, 129, 64, 64]
    cu = np.concatenate([[0], np.cumsum(lens)])
    N, H = int(cu[-1]), 4
    q, k, v = (torch.randn(N, H, D, generator=g).bfloat16() for _ in range(3))
    want = enc.encoder_attention_ref(q.float(), k.float(), v.float(), cu, D ** -0.5)
    plan = enc.make_plan(cu, DEV)
    got = enc.encoder_attention(q.to(DEV), k.to(DEV), v.to(DEV), plan, D ** -0.5)
    torch.cuda.synchronize()
    _native.check_status(torch.device(DEV))
    assert got.shape == (N, H, D)
    assert (got.float().cpu() - want).abs().max() < 3e-2


def test_vision_tower_on_gpu_matches_fp32():
    from vllm_ascend_b200.models.vision import VisionConfig, VisionTransformer
    cfg = VisionConfig(depth=3, hidden_size=256, num_heads=4, intermediate_size=512, out_hidden_size=256,
                       window_size=112, fullatt_block_indexes=[2], init_std=0.05)
    cpu = VisionTransformer(cfg, "cpu", torch.float32)
    gpu = VisionTransformer(cfg, DEV, torch.bfloat16)
    gpu.load_weights([(n, t) for n, t in cpu.named_parameters()])
    grid = np.array([[1, 16, 20], [2, 8, 8]])
    n = int((grid[:, 0] * grid[:, 1] * grid[:, 2]).sum())
    px = torch.randn(n, cfg.patch_dim, generator=torch.Generator().manual_seed(3))
    want = cpu(px, grid)
    c0 = _native.launch_counter[0]
    got = gpu(px.to(DEV), grid).float().cpu()
    assert _native.launch_counter[0] - c0 >= 9 * cfg.depth        # native kernels, not a fallback
    _native.check_status(torch.device(DEV))
    rel = (got - want).norm() / want.norm()
    assert rel < 3e-2, rel


def test_vision_language_engine_on_gpu():
    """Graph decode equals eager decode, and image content changes the continuation."""
    from vllm_ascend_b200.config import ModelConfig
    from vllm_ascend_b200.engine.llm import LLM
    from vllm_ascend_b200.engine.request import SamplingParams

    def cfg():
        return ModelConfig(name="vl-t", architecture="Qwen2_5_VLForConditionalGeneration", vocab_size=2048,
                           hidden_size=512, intermediate_size=1024, num_hidden_layers=3, num_attention_heads=8,
                           num_key_value_heads=2, head_dim=128, attention_bias=True, rope_theta=1e6,
                           dtype="bfloat16", init_std=0.05, mrope_section=[16, 24, 24], image_token_id=2000,
                           video_token_id=2001,
                           vision_config=dict(depth=2, hidden_size=256, num_heads=4, intermediate_size=512,
                                              out_hidden_size=512, window_size=112, fullatt_block_indexes=[1],
                                              init_std=0.05))
    g = torch.Generator().manual_seed(0)
    grid = (1, 16, 12)
    img_a = torch.randn(16 * 12, 3 * 2 * 14 * 14, generator=g)
    img_b = torch.randn(16 * 12, 3 * 2 * 14 * 14, generator=g)
    rng = np.random.default_rng(0)
    text = rng.integers(0, 1900, size=40).tolist()
    ids = text[:10] + [2000] + text[10:]

    def prompts(img):
        return [{"prompt_token_ids": ids, "multi_modal_data": {"image": [(img, grid)]}},
                {"prompt_token_ids": text}]
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    outs = {}
    for eager in (True, False):
        llm = LLM(cfg(), device="cuda", max_model_len=512, max_num_seqs=8, max_num_batched_tokens=64,
                  num_gpu_blocks_override=40, enforce_eager=eager, cudagraph_capture_sizes=[2, 4])
        outs[eager] = [o.outputs[0].token_ids for o in llm.generate(prompts(img_a), sp)]
        if eager:
            other = [o.outputs[0].token_ids for o in llm.generate(prompts(img_b), sp)]
            assert other[1] == outs[eager][1]              # the text-only request ignores images
            assert other[0] != outs[eager][0]
            assert llm.engine.runner.mm.stats["encoder_items"] == 2
        else:
            assert llm.engine.runner.stats["graph_replays"] > 0
            assert llm.engine.runner.mm.encoder_graphs.stats["replays"] == 1
    assert outs[True] == outs[False]
    _native.check_status(torch.device("cuda"))


def test_encoder_graph_replay_matches_eager():
    from vllm_ascend_b200.compilation.encoder_graph import EncoderGraphManager
    from vllm_ascend_b200.models.vision import VisionConfig, VisionTransformer
    cfg = VisionConfig(depth=2, hidden_size=256, num_heads=4, intermediate_size=512, out_hidden_size=256,
                       window_size=112, fullatt_block_indexes=[1], init_std=0.05)
    tower = VisionTransformer(cfg, DEV, torch.bfloat16)
    mgr = EncoderGraphManager(tower, bucket_sizes=(512, 2048))
    g = torch.Generator().manual_seed(5)
    for grid in ([[1, 16, 20]], [[1, 8, 8], [1, 12, 16]], [[1, 16, 20]], [[2, 24, 28]]):
        grid = np.array(grid)
        n = int((grid[:, 0] * grid[:, 1] * grid[:, 2]).sum())
        px = torch.randn(n, cfg.patch_dim, generator=g).to(DEV).bfloat16()
        want = tower(px, grid).float()
        got = mgr.run(px, grid).float()
        assert got.shape == want.shape
        assert (got - want).abs().max() < 2e-2 * want.abs().max()
    assert mgr.stats["captures"] == 2 and mgr.stats["replays"] == 4
    _native.check_status(torch.device(DEV))


@pytest.mark.parametrize("H,T", [(1152, 300), (4608, 77), (64, 5), (10240, 3)])
def test_layer_norm_kernel(H, T):
    g = torch.Generator().manual_seed(4)
    x = (torch.randn(T, H, generator=g) * 2 + 0.7).bfloat16()
    w, b = (torch.rand(H, generator=g) + 0.5).bfloat16(), torch.randn(H, generator=g).bfloat16()
    want = torch.nn.functional.layer_norm(x.float(), (H,), w.float(), b.float(), 1e-6)
    c0 = _native.launch_counter[0]
    got = ops.layer_norm(x.to(DEV), w.to(DEV), b.to(DEV), 1e-6)
    assert _native.launch_counter[0] == c0 + 1
    assert (got.float().cpu() - want).abs().max() < 4e-2
    nob = ops.layer_norm(x.to(DEV), w.to(DEV), None, 1e-6)
    want0 = torch.nn.functional.layer_norm(x.float(), (H,), w.float(), None, 1e-6)
    assert (nob.float().cpu() - want0).abs().max() < 4e-2


def test_qwen3_vl_tower_on_gpu_matches_fp32():
    from vllm_ascend_b200.models.vision import Qwen3VisionTransformer, VisionConfig
    cfg = VisionConfig(depth=3, hidden_size=288, num_heads=4, intermediate_size=512, out_hidden_size=256,
                       patch_size=16, num_position_embeddings=64, deepstack_visual_indexes=[0, 2], init_std=0.05)
    cpu = Qwen3VisionTransformer(cfg, "cpu", torch.float32)
    gpu = Qwen3VisionTransformer(cfg, DEV, torch.bfloat16)
    gpu.load_weights([(n, t) for n, t in cpu.named_parameters()])
    grid = np.array([[1, 16, 20], [2, 8, 8]])
    n = int((grid[:, 0] * grid[:, 1] * grid[:, 2]).sum())
    px = torch.randn(n, cfg.patch_dim, generator=torch.Generator().manual_seed(3))
    want = cpu(px, grid)
    c0 = _native.launch_counter[0]
    got = gpu(px.to(DEV), grid).float().cpu()
    assert _native.launch_counter[0] - c0 >= 10 * cfg.depth
    _native.check_status(torch.device(DEV))
    assert got.shape == want.shape == (n // 4, 3 * 256)
    for i in range(3):
        a, b = got[:, 256 * i:256 * (i + 1)], want[:, 256 * i:256 * (i + 1)]
        assert (a - b).norm() / b.norm() < 3e-2, i


def test_qwen3_vl_engine_on_gpu():
    """Deepstack rows under CUDA-graph decode and chunked prefill: graph output equals eager, and the
    image changes the continuation."""
    from vllm_ascend_b200.config import ModelConfig
    from vllm_ascend_b200.engine.llm import LLM
    from vllm_ascend_b200.engine.request import SamplingParams

    def cfg():
        return ModelConfig(name="vl3-t", architecture="Qwen3VLForConditionalGeneration", vocab_size=2048,
                           hidden_size=512, intermediate_size=1024, num_hidden_layers=3, num_attention_heads=8,
                           num_key_value_heads=2, head_dim=128, qk_norm=True, rope_theta=1e6,
                           dtype="bfloat16", init_std=0.05, mrope_section=[24, 20, 20], mrope_interleaved=True,
                           image_token_id=2000, video_token_id=2001,
                           vision_config=dict(depth=2, hidden_size=256, num_heads=4, intermediate_size=512,
                                              out_hidden_size=512, patch_size=16, num_position_embeddings=64,
                                              deepstack_visual_indexes=[0, 1], init_std=0.05))
    g = torch.Generator().manual_seed(0)
    grid = (1, 16, 12)
    img_a = torch.randn(16 * 12, 3 * 2 * 16 * 16, generator=g)
    img_b = torch.randn(16 * 12, 3 * 2 * 16 * 16, generator=g)
    rng = np.random.default_rng(0)
    text = rng.integers(0, 1900, size=40).tolist()
    ids = text[:10] + [2000] + text[10:]
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    outs = {}
    for eager in (True, False):
        llm = LLM(cfg(), device="cuda", max_model_len=512, max_num_seqs=8, max_num_batched_tokens=64,
                  num_gpu_blocks_override=40, enforce_eager=eager, cudagraph_capture_sizes=[2, 4])
        assert llm.engine.runner.model.num_deepstack == 2
        outs[eager] = llm.generate([{"prompt_token_ids": ids, "multi_modal_data": {"image": [(img_a, grid)]}}],
                                   sp)[0].outputs[0].token_ids
        if eager:
            other = llm.generate([{"prompt_token_ids": ids, "multi_modal_data": {"image": [(img_b, grid)]}}],
                                 sp)[0].outputs[0].token_ids
            assert other != outs[eager]
    assert outs[True] == outs[False]
    _native.check_status(torch.device("cuda"))


def test_audio_tower_on_gpu_matches_fp32():
    from vllm_ascend_b200.models.audio import AudioConfig, AudioEncoder, audio_output_lengths
    cfg = AudioConfig(num_mel_bins=128, d_model=256, encoder_layers=2, encoder_attention_heads=4, encoder_ffn_dim=512,
                      max_source_positions=300, init_std=0.05, output_dim=384)
    cpu = AudioEncoder(cfg, "cpu", torch.float32)
    gpu = AudioEncoder(cfg, DEV, torch.bfloat16)
    for (n, a), (_, b) in zip(cpu.named_parameters(), gpu.named_parameters()):
        b.copy_(a)
    g = torch.Generator().manual_seed(5)
    feats = [torch.randn(128, 600, generator=g), torch.randn(128, 600, generator=g)]
    valid = [600, 333]
    want = cpu(feats, valid)
    c0 = _native.launch_counter[0]
    got = gpu([f.to(DEV) for f in feats], valid).float().cpu()
    assert _native.launch_counter[0] - c0 >= 6 * cfg.encoder_layers + 6     # native kernels, not a fallback
    _native.check_status(torch.device(DEV))
    assert got.shape == want.shape == (int(audio_output_lengths(valid)[1].sum()), 384)
    assert (got - want).norm() / want.norm() < 3e-2
