"""Vision tower, multimodal rotary positions and the multimodal engine path on CPU.
The oracle for the tower is the transformers implementation with the same weights."""
import numpy as np
import pytest
import torch

from vllm_ascend_b200.models.vision import VisionConfig, VisionTransformer, window_index


def _hf_tower(cfg: VisionConfig):
    from transformers.models.qwen2_5_vl.configuration_qwen2_5_vl import Qwen2_5_VLVisionConfig
    from transformers.models.qwen2_5_vl.modeling_qwen2_5_vl import Qwen2_5_VisionTransformerPretrainedModel
    hc = Qwen2_5_VLVisionConfig(depth=cfg.depth, hidden_size=cfg.hidden_size, num_heads=cfg.num_heads,
                                intermediate_size=cfg.intermediate_size, out_hidden_size=cfg.out_hidden_size,
                                patch_size=cfg.patch_size, spatial_merge_size=cfg.spatial_merge_size,
                                temporal_patch_size=cfg.temporal_patch_size, window_size=cfg.window_size,
                                fullatt_block_indexes=cfg.fullatt_block_indexes, in_channels=cfg.in_channels)
    hc._attn_implementation = "eager"
    torch.manual_seed(0)
    m = Qwen2_5_VisionTransformerPretrainedModel(hc).eval().float()
    with torch.no_grad():
        for p in m.parameters():
            p.normal_(0, 0.05)
    return m


def test_vision_tower_matches_transformers():
    cfg = VisionConfig(depth=3, hidden_size=64, num_heads=4, intermediate_size=96, out_hidden_size=48,
                       patch_size=14, window_size=56, fullatt_block_indexes=[1])
    hf = _hf_tower(cfg)
    ours = VisionTransformer(cfg, "cpu", torch.float32)
    loaded = ours.load_weights(hf.state_dict().items())
    assert len(loaded) == len(hf.state_dict())
    grid = np.array([[1, 6, 8], [2, 4, 4], [1, 10, 6]])
    n = int((grid[:, 0] * grid[:, 1] * grid[:, 2]).sum())
    px = torch.randn(n, cfg.patch_dim, generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        ref = hf(px, grid_thw=torch.from_numpy(grid))
    ref = ref.pooler_output if hasattr(ref, "pooler_output") else ref
    got = ours(px, grid)
    assert got.shape == ref.shape == (n // 4, 48)
    assert torch.allclose(got, ref, atol=2e-4, rtol=2e-4), (got - ref).abs().max()


def test_window_index_is_a_permutation_with_full_coverage():
    grid = np.array([[2, 6, 10], [1, 4, 4]])
    idx, cu = window_index(grid, 56, 2, 14)
    total = int((grid[:, 0] * (grid[:, 1] // 2) * (grid[:, 2] // 2)).sum())
    assert sorted(idx.tolist()) == list(range(total))
    assert cu[0] == 0 and cu[-1] == total * 4 and (np.diff(cu) > 0).all()


def _hf_vl():
    from transformers.models.qwen2_5_vl.configuration_qwen2_5_vl import Qwen2_5_VLConfig
    from transformers.models.qwen2_5_vl.modeling_qwen2_5_vl import Qwen2_5_VLForConditionalGeneration
    cfg = Qwen2_5_VLConfig(
        text_config=dict(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                         num_attention_heads=4, num_key_value_heads=2, rope_theta=1e6,
                         rope_scaling={"type": "mrope", "mrope_section": [4, 6, 6]},
                         max_position_embeddings=2048, tie_word_embeddings=False),
        vision_config=dict(depth=2, hidden_size=64, num_heads=4, intermediate_size=96, out_hidden_size=128,
                           patch_size=14, window_size=56, fullatt_block_indexes=[1]),
        image_token_id=500, video_token_id=501, vision_start_token_id=502, vision_end_token_id=503)
    cfg._attn_implementation = "eager"
    cfg.architectures = ["Qwen2_5_VLForConditionalGeneration"]
    torch.manual_seed(0)
    m = Qwen2_5_VLForConditionalGeneration(cfg).eval().float()
    with torch.no_grad():
        for p in m.parameters():
            p.normal_(0, 0.05)
        for n, p in m.named_parameters():
            if "norm" in n or "ln_q" in n:
                p.fill_(1.0)
    return cfg, m


def _mm_prompt(rng):
    """text, image (1x4x6 patches -> 6 tokens), text, image (1x8x4 -> 8 tokens), text."""
    grids = [(1, 4, 6), (1, 8, 4)]
    px = [torch.randn(g[0] * g[1] * g[2], 3 * 2 * 14 * 14, generator=rng) for g in grids]
    ids = [3, 4, 5, 502, 500, 503, 7, 8, 9, 10, 502, 500, 503, 11, 12]
    return ids, px, grids


def test_mrope_positions_match_transformers():
    from vllm_ascend_b200.multimodal import expand_placeholders, mrope_positions
    from vllm_ascend_b200.multimodal.inputs import MMInput
    cfg, hf = _hf_vl()
    ids, px, grids = _mm_prompt(torch.Generator().manual_seed(0))
    lengths = [g[0] * g[1] * g[2] // 4 for g in grids]
    full, offs = expand_placeholders(ids, 500, lengths)
    items = [MMInput("image", o, n, g, None) for o, n, g in zip(offs, lengths, grids)]
    got, delta = mrope_positions(full, items, 2, 2.0)
    t = torch.tensor([full])
    want, want_delta = hf.model.get_rope_index(t, mm_token_type_ids=(t == 500).int(),
                                               image_grid_thw=torch.tensor(grids))
    want = want[:, 0].numpy()
    # height / width axes and every text position agree with transformers; the temporal axis of an
    # image follows the published rule (all frame groups of an image sit at the item's start
    # position), which this transformers version scales differently
    assert np.array_equal(got[1:], want[1:])
    text = np.array(full) != 500
    assert np.array_equal(got[0][text], want[0][text])
    for it in items:
        assert (got[0, it.offset:it.end] == got[1, it.offset]).all()
    assert delta == got.max() + 1 - len(full) == -7


def test_multimodal_engine_matches_transformers_greedy():
    """Images through the vision tower, merged embeddings, 3-axis rotary positions, chunked prefill
    and decode: the engine's greedy tokens equal transformers' on the same weights."""
    from vllm_ascend_b200.config import ModelConfig
    from vllm_ascend_b200.engine.llm import LLM
    from vllm_ascend_b200.engine.request import SamplingParams
    cfg, hf = _hf_vl()
    mcfg = ModelConfig.from_hf_dict(cfg.to_dict(), dtype="float32", architecture="Qwen2_5_VLForConditionalGeneration")
    assert mcfg.mrope_section == [4, 6, 6] and mcfg.is_multimodal and mcfg.image_token_id == 500
    llm = LLM(mcfg, device="cpu", max_model_len=256, max_num_seqs=4, max_num_batched_tokens=16,
              num_gpu_blocks_override=64, block_size=16)
    loaded = llm.engine.runner.model.load_weights(hf.state_dict().items())
    assert len(loaded) == len(hf.state_dict())
    ids, px, grids = _mm_prompt(torch.Generator().manual_seed(0))
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    outs = llm.generate([{"prompt_token_ids": ids, "multi_modal_data": {"image": list(zip(px, grids))}},
                         {"prompt_token_ids": [9, 8, 7, 6, 5]}], sp)
    # oracle: greedy decoding by full recomputation with the same 3-axis positions
    from vllm_ascend_b200.multimodal import mrope_positions
    full = outs[0].prompt_token_ids
    assert len(full) == len(ids) - 2 + 6 + 8
    from vllm_ascend_b200.multimodal import build_mm_request
    _, req_items = build_mm_request(ids, {"image": list(zip(px, grids))}, mcfg)
    pos, delta = mrope_positions(full, req_items, 2, 2.0)

    def greedy(seq, pos3, **kw):
        out = []
        seq = list(seq)
        for _ in range(6):
            L = len(seq)
            p3 = np.concatenate([pos3, np.arange(pos3.shape[1], L)[None].repeat(3, 0) + kw.get("delta", 0)], axis=1)
            t = torch.tensor([seq])
            with torch.no_grad():
                lg = hf(input_ids=t, position_ids=torch.from_numpy(p3)[:, None, :], attention_mask=torch.ones_like(t),
                        **{k: v for k, v in kw.items() if k != "delta"}).logits
            seq.append(int(lg[0, -1].argmax()))
            out.append(seq[-1])
        return out
    want = greedy(full, pos, delta=delta, pixel_values=torch.cat(px), image_grid_thw=torch.tensor(grids))
    assert outs[0].outputs[0].token_ids == want
    txt = [9, 8, 7, 6, 5]
    assert outs[1].outputs[0].token_ids == greedy(txt, np.arange(5)[None].repeat(3, 0))
    mm = llm.engine.runner.mm
    assert mm.stats["encoder_items"] == 2 and not mm.encoder_cache      # outputs dropped after use


def test_disaggregated_encoder_through_ec_store():
    """Encoder instance publishes outputs by content hash; the serving instance gets the request with
    hashes only (no pixels) and produces the tokens of a monolithic run."""
    from vllm_ascend_b200.distributed.kv_transfer.kv_pool import KVStoreServer
    from vllm_ascend_b200.engine.llm import LLM
    from vllm_ascend_b200.engine.request import SamplingParams
    store = KVStoreServer()
    try:
        def mk(role=None):
            ec = None if role is None else {"ec_connector": "ECStoreConnector", "ec_role": role,
                                            "ec_connector_extra_config": {"store_port": store.port}}
            return LLM("tiny-vl", device="cpu", max_model_len=256, max_num_seqs=4, max_num_batched_tokens=32,
                       num_gpu_blocks_override=64, block_size=16, ec_transfer_config=ec)
        ids, px, grids = _mm_prompt(torch.Generator().manual_seed(0))
        ids = [t for t in ids if t not in (502, 503)]
        sp = SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True)
        mono = mk().generate([{"prompt_token_ids": ids, "multi_modal_data": {"image": list(zip(px, grids))}}], sp)
        enc_inst = mk("ec_producer")
        descs = enc_inst.encode_multimodal({"image": list(zip(px, grids))})
        assert [d["grid_thw"] for d in descs] == [list(g) for g in grids]
        assert enc_inst.engine.runner.mm.ec_connector.stats["saved"] == 2
        pd = mk("ec_consumer")
        outs = pd.generate([{"prompt_token_ids": ids, "multi_modal_data": {"image": [
            {"hash": d["hash"], "grid_thw": d["grid_thw"]} for d in descs]}}], sp)
        assert outs[0].outputs[0].token_ids == mono[0].outputs[0].token_ids
        mm = pd.engine.runner.mm
        assert mm.stats["remote_items"] == 2 and mm.stats["encoder_runs"] == 0
        # a miss with no pixels is an error the caller sees, not a silent zero embedding
        with pytest.raises(RuntimeError):
            pd.generate([{"prompt_token_ids": ids, "multi_modal_data": {"image": [
                {"hash": "0" * 32, "grid_thw": list(grids[0])}, {"hash": "1" * 32, "grid_thw": list(grids[1])}]}}], sp)
    finally:
        store.close()


def test_patchify_layout_and_resize():
    from vllm_ascend_b200.multimodal import patchify, smart_resize
    assert smart_resize(100, 200, 28) == (112, 196)
    img = (np.random.default_rng(0).random((56, 84, 3)) * 255).astype(np.uint8)
    pv, (t, gh, gw) = patchify(img, normalize=False)
    assert (t, gh, gw) == (1, 4, 6) and pv.shape == (24, 3 * 2 * 14 * 14)
    # row 0 is the top-left patch, row 1 its right neighbour, row 2 the patch below row 0 (2x2 merge groups)
    x = img.astype(np.float32) / 255
    first = pv[0].reshape(3, 2, 14, 14)
    assert np.allclose(first[:, 0], x[:14, :14].transpose(2, 0, 1), atol=1e-6)
    assert np.allclose(first[:, 1], first[:, 0])                 # single image repeated over the temporal patch
    assert np.allclose(pv[1].reshape(3, 2, 14, 14)[:, 0], x[:14, 14:28].transpose(2, 0, 1), atol=1e-6)
    assert np.allclose(pv[2].reshape(3, 2, 14, 14)[:, 0], x[14:28, :14].transpose(2, 0, 1), atol=1e-6)
    assert np.allclose(pv[4].reshape(3, 2, 14, 14)[:, 0], x[:14, 28:42].transpose(2, 0, 1), atol=1e-6)


# ---------------------------------------------------------------- Qwen3-VL (deepstack, learned positions)
def _hf_qwen3_vl():
    from transformers import Qwen3VLConfig, Qwen3VLForConditionalGeneration
    cfg = Qwen3VLConfig(
        text_config=dict(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=3,
                         num_attention_heads=4, num_key_value_heads=2, head_dim=32,
                         rope_parameters={"rope_type": "default", "rope_theta": 1e6, "mrope_section": [4, 6, 6],
                                          "mrope_interleaved": True},
                         max_position_embeddings=2048, tie_word_embeddings=False),
        vision_config=dict(depth=3, hidden_size=64, num_heads=4, intermediate_size=96, out_hidden_size=128,
                           patch_size=14, num_position_embeddings=36, deepstack_visual_indexes=[0, 1]),
        image_token_id=500, video_token_id=501, vision_start_token_id=502, vision_end_token_id=503)
    cfg._attn_implementation = "eager"
    cfg.architectures = ["Qwen3VLForConditionalGeneration"]
    torch.manual_seed(0)
    m = Qwen3VLForConditionalGeneration(cfg).eval().float()
    with torch.no_grad():
        for n, p in m.named_parameters():
            p.normal_(0, 0.05)
            if "norm" in n and n.endswith("weight"):
                p.add_(1.0)
    return cfg, m


def test_qwen3_vl_tower_matches_transformers():
    from vllm_ascend_b200.models.vision import Qwen3VisionTransformer
    cfg, hf = _hf_qwen3_vl()
    vc = VisionConfig.from_hf(cfg.vision_config.to_dict())
    assert vc.num_position_embeddings == 36 and vc.deepstack_visual_indexes == [0, 1]
    ours = Qwen3VisionTransformer(vc, "cpu", torch.float32)
    sd = hf.model.visual.state_dict()
    assert len(ours.load_weights(sd.items())) == len(sd)
    grid = np.array([[1, 6, 8], [2, 4, 4], [1, 10, 6]])
    n = int((grid[:, 0] * grid[:, 1] * grid[:, 2]).sum())
    px = torch.randn(n, vc.patch_dim, generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        ref = hf.model.visual(px, grid_thw=torch.from_numpy(grid))
    main = ref.pooler_output if hasattr(ref, "pooler_output") else ref[0]
    deep = ref.deepstack_features if hasattr(ref, "deepstack_features") else ref[1]
    got = ours(px, grid)
    assert got.shape == (n // 4, 3 * 128)
    assert torch.allclose(got[:, :128], main, atol=2e-4, rtol=2e-4), (got[:, :128] - main).abs().max()
    for i, d in enumerate(deep):
        assert torch.allclose(got[:, 128 * (i + 1):128 * (i + 2)], d, atol=2e-4, rtol=2e-4)


def test_qwen3_vl_engine_matches_transformers_greedy():
    """Deepstack features join the residual stream after the first decoder layers, positions use the
    interleaved 3-axis rotary layout: greedy tokens equal transformers' under chunked prefill."""
    from vllm_ascend_b200.config import ModelConfig
    from vllm_ascend_b200.engine.llm import LLM
    from vllm_ascend_b200.engine.request import SamplingParams
    from vllm_ascend_b200.multimodal import build_mm_request, mrope_positions
    cfg, hf = _hf_qwen3_vl()
    mcfg = ModelConfig.from_hf_dict(cfg.to_dict(), dtype="float32", architecture="Qwen3VLForConditionalGeneration")
    assert mcfg.mrope_section == [4, 6, 6] and mcfg.mrope_interleaved and mcfg.qk_norm
    llm = LLM(mcfg, device="cpu", max_model_len=256, max_num_seqs=4, max_num_batched_tokens=16,
              num_gpu_blocks_override=64, block_size=16)
    loaded = llm.engine.runner.model.load_weights(hf.state_dict().items())
    assert len(loaded) == len(hf.state_dict())
    ids, px, grids = _mm_prompt(torch.Generator().manual_seed(0))
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    outs = llm.generate([{"prompt_token_ids": ids, "multi_modal_data": {"image": list(zip(px, grids))}},
                         {"prompt_token_ids": [9, 8, 7, 6, 5]}], sp)
    full = outs[0].prompt_token_ids
    _, items = build_mm_request(ids, {"image": list(zip(px, grids))}, mcfg)
    pos, delta = mrope_positions(full, items, 2, 2.0)
    seq, want = list(full), []
    for _ in range(6):
        L = len(seq)
        p3 = np.concatenate([pos, np.arange(pos.shape[1], L)[None].repeat(3, 0) + delta], axis=1)
        t = torch.tensor([seq])
        with torch.no_grad():
            lg = hf(input_ids=t, position_ids=torch.from_numpy(p3)[:, None, :], attention_mask=torch.ones_like(t),
                    pixel_values=torch.cat(px), image_grid_thw=torch.tensor(grids)).logits
        seq.append(int(lg[0, -1].argmax()))
        want.append(seq[-1])
    assert outs[0].outputs[0].token_ids == want


# ---------------------------------------------------------------- audio-language model (Qwen2-Audio layout)
def _hf_audio_lm():
    from transformers import Qwen2AudioConfig, Qwen2AudioForConditionalGeneration
    cfg = Qwen2AudioConfig(
        audio_config=dict(num_mel_bins=16, d_model=64, encoder_layers=2, encoder_attention_heads=4, encoder_ffn_dim=128,
                          max_source_positions=50),
        text_config=dict(model_type="qwen2", vocab_size=512, hidden_size=128, intermediate_size=256,
                         num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, rope_theta=1e6,
                         max_position_embeddings=2048, tie_word_embeddings=False),
        audio_token_index=500)
    cfg._attn_implementation = "eager"
    cfg.architectures = ["Qwen2AudioForConditionalGeneration"]
    torch.manual_seed(0)
    m = Qwen2AudioForConditionalGeneration(cfg).eval().float()
    with torch.no_grad():
        for n, p in m.named_parameters():
            p.normal_(0, 0.05)
            if "norm" in n and n.endswith("weight"):
                p.add_(1.0)
    return cfg, m


def test_audio_language_engine_matches_transformers_greedy():
    """Two padded clips of different valid lengths: conv front end as GEMMs, attention over the
    valid frames only, pair pooling, projector, merge into the prompt; greedy tokens equal
    transformers' under chunked prefill."""
    from vllm_ascend_b200.config import ModelConfig
    from vllm_ascend_b200.engine.llm import LLM
    from vllm_ascend_b200.engine.request import SamplingParams
    from vllm_ascend_b200.models.audio import audio_output_lengths
    cfg, hf = _hf_audio_lm()
    mcfg = ModelConfig.from_hf_dict(cfg.to_dict(), dtype="float32", architecture="Qwen2AudioForConditionalGeneration")
    assert mcfg.is_multimodal and mcfg.audio_token_id == 500 and mcfg.audio_config["d_model"] == 64
    llm = LLM(mcfg, device="cpu", max_model_len=256, max_num_seqs=4, max_num_batched_tokens=16,
              num_gpu_blocks_override=64, block_size=16)
    loaded = llm.engine.runner.model.load_weights(hf.state_dict().items())
    assert len(loaded) == len(hf.state_dict())
    g = torch.Generator().manual_seed(0)
    feats = [torch.randn(16, 100, generator=g), torch.randn(16, 100, generator=g)]
    valid = [100, 57]
    n_tok = [int(x) for x in audio_output_lengths(valid)[1]]
    assert n_tok == [25, 14]
    ids = [3, 4, 500, 7, 8, 9, 500, 11, 12]
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    outs = llm.generate([{"prompt_token_ids": ids, "multi_modal_data": {"audio": list(zip(feats, valid))}},
                         {"prompt_token_ids": [9, 8, 7, 6, 5]}], sp)
    full = outs[0].prompt_token_ids
    assert len(full) == len(ids) - 2 + sum(n_tok)
    mask = torch.zeros(2, 100, dtype=torch.long)
    mask[0, :100], mask[1, :57] = 1, 1
    seq, want = list(full), []
    for _ in range(6):
        t = torch.tensor([seq])
        with torch.no_grad():
            lg = hf(input_ids=t, attention_mask=torch.ones_like(t), input_features=torch.stack(feats),
                    feature_attention_mask=mask).logits
        seq.append(int(lg[0, -1].argmax()))
        want.append(seq[-1])
    assert outs[0].outputs[0].token_ids == want
    assert llm.engine.runner.mm.stats["encoder_items"] == 2
