"""Vision tower, multimodal rotary positions and the vision-language forward pass against the
HuggingFace implementation of Qwen2.5-VL (random small configuration, CPU, fp32)."""
import pytest
import torch

transformers = pytest.importorskip("transformers")


def _hf():
    from transformers import Qwen2_5_VLConfig, Qwen2_5_VLForConditionalGeneration
    torch.manual_seed(0)
    cfg = Qwen2_5_VLConfig(
        text_config=dict(vocab_size=1024, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                         num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=512,
                         rope_scaling={"type": "mrope", "mrope_section": [4, 6, 6]}, rope_theta=10000.0),
        vision_config=dict(depth=3, hidden_size=64, intermediate_size=96, num_heads=4, patch_size=14, spatial_merge_size=2,
                           temporal_patch_size=2, out_hidden_size=128, window_size=56, fullatt_block_indexes=[1],
                           # one position step per temporal grid step: still images then sit at their start position,
                           # the published Qwen2.5-VL behaviour
                           tokens_per_second=1),
        image_token_id=1000, video_token_id=1001, vision_start_token_id=1002, vision_end_token_id=1003)
    m = Qwen2_5_VLForConditionalGeneration(cfg).eval().float()
    for p in m.parameters():                              # biases and norms away from their trivial initial values
        if p.dim() == 1:
            torch.nn.init.normal_(p, mean=0.5, std=0.2)
    return cfg, m


def _arch(cfg):
    from chatlearn_b200.models.nn.arch import ModelArch
    return ModelArch.from_hf_dict(cfg.to_dict())


def test_vision_tower_matches_hf():
    from chatlearn_b200.models.nn.vision import VisionArch, VisionTower
    cfg, hf = _hf()
    va = VisionArch.from_hf_dict(cfg.vision_config.to_dict())
    tower = VisionTower(va)
    tower.load_hf_state_dict(hf.state_dict())
    grid = torch.tensor([[1, 6, 8], [1, 4, 4], [1, 10, 6]])             # windows of 2x2 merge groups: ragged edges
    n = int((grid[:, 0] * grid[:, 1] * grid[:, 2]).sum())
    px = torch.randn(n, va.patch_dim)
    with torch.no_grad():
        want = hf.model.visual(px, grid_thw=grid).pooler_output
        got = tower(px, grid)
    assert got.shape == want.shape == (n // 4, 128)
    assert torch.allclose(got, want, rtol=1e-4, atol=1e-4), (got - want).abs().max()


def test_mrope_positions_match_hf():
    from chatlearn_b200.models.nn.vision import mrope_positions
    cfg, hf = _hf()
    grid = torch.tensor([[1, 6, 8], [1, 4, 4]])
    ids = [5, 6, 1002] + [1000] * 12 + [1003, 7, 8, 9, 1002] + [1000] * 4 + [1003, 10, 11]
    input_ids = torch.tensor([ids])
    mm = (input_ids == 1000).long()
    want, delta = hf.model.get_rope_index(input_ids, mm_token_type_ids=mm, image_grid_thw=grid)
    got, d = mrope_positions(input_ids[0], grid, 1000, 2)
    assert torch.equal(got, want[:, 0]) and d == int(delta[0])


def test_full_forward_logits_match_hf():
    from chatlearn_b200.models.nn.model import packed_ctx
    from chatlearn_b200.models.nn.vl_model import VLCausalLM
    cfg, hf = _hf()
    arch = _arch(cfg)
    assert arch.mrope_section == [4, 6, 6] and arch.image_token_id == 1000 and arch.attention_bias
    model = VLCausalLM(arch)
    model.load_hf_state_dict(hf.state_dict())
    grid = torch.tensor([[1, 6, 8]])
    ids = torch.tensor([3, 4, 1002] + [1000] * 12 + [1003, 20, 21, 22, 23])
    px = torch.randn(48, model.varch.patch_dim)
    with torch.no_grad():
        want = hf(input_ids=ids[None], pixel_values=px, image_grid_thw=grid, mm_token_type_ids=(ids[None] == 1000).long()).logits[0]
        ctx, _ = packed_ctx([ids.numel()], "cpu")
        ctx.mrope_positions = model.positions(ids, grid)
        got = model.logits(ids, ctx, px, grid)
    assert torch.allclose(got, want, rtol=2e-4, atol=2e-4), (got - want).abs().max()
    # two sequences packed into one row: each keeps its own positions and attends only to itself
    ids2 = torch.tensor([9, 8, 7, 6])
    with torch.no_grad():
        want2 = hf(input_ids=ids2[None]).logits[0]
        ctx, _ = packed_ctx([ids.numel(), ids2.numel()], "cpu")
        ctx.mrope_positions = model.packed_positions([ids, ids2], [grid, None])
        both = model.logits(torch.cat([ids, ids2]), ctx, px, grid)
    assert torch.allclose(both[:ids.numel()], want, rtol=2e-4, atol=2e-4)
    assert torch.allclose(both[ids.numel():], want2, rtol=2e-4, atol=2e-4)


def test_image_patches_match_hf_processor():
    import numpy as np
    from PIL import Image
    from transformers import Qwen2VLImageProcessor
    from chatlearn_b200.data.vision_utils import expand_image_tokens, image_to_patches, smart_resize
    rng = np.random.default_rng(0)
    img = Image.fromarray(rng.integers(0, 255, (75, 131, 3), dtype=np.uint8))
    proc = Qwen2VLImageProcessor(min_pixels=56 * 56, max_pixels=28 * 28 * 64)
    want = proc(images=[img], return_tensors="pt")
    got, grid = image_to_patches(img, min_pixels=56 * 56, max_pixels=28 * 28 * 64)
    assert list(grid) == want["image_grid_thw"][0].tolist()
    assert got.shape == want["pixel_values"].shape
    assert torch.allclose(got, want["pixel_values"], atol=2e-2), (got - want["pixel_values"]).abs().max()
    assert smart_resize(75, 131, 28, 56 * 56, 28 * 28 * 64) == (grid[1] * 14, grid[2] * 14)
    ids = expand_image_tokens([1, 1000, 2], [grid], 1000)
    assert ids.count(1000) == grid[1] * grid[2] // 4 and ids[0] == 1 and ids[-1] == 2


def test_rollout_engine_generates_like_hf_with_an_image():
    from chatlearn_b200.models.nn.model import CausalLM
    from chatlearn_b200.models.nn.vision import VisionArch, VisionTower
    from chatlearn_b200.models.nn.vl_model import strip_language_prefix
    from chatlearn_b200.rollout import RolloutEngine, SamplingParams
    cfg, hf = _hf()
    arch = _arch(cfg)
    arch.eos_token_id = 1023
    lm = CausalLM(arch)
    lm.load_hf_state_dict(strip_language_prefix(hf.state_dict()))
    tower = VisionTower(VisionArch.from_hf_dict(cfg.vision_config.to_dict()))
    tower.load_hf_state_dict(hf.state_dict())
    eng = RolloutEngine(lm, block_size=8, num_blocks=64, max_num_seqs=4, max_num_batched_tokens=64, max_model_len=128,
                        vision=tower)
    grid = torch.tensor([[1, 6, 8]])
    ids = [3, 4, 1002] + [1000] * 12 + [1003, 20, 21, 22, 23]
    px = torch.randn(48, tower.arch.patch_dim)
    text_only = [9, 8, 7, 6, 5]
    new = 8
    with torch.no_grad():
        want = hf.generate(input_ids=torch.tensor([ids]), pixel_values=px, image_grid_thw=grid,
                           mm_token_type_ids=(torch.tensor([ids]) == 1000).long(),
                           max_new_tokens=new, do_sample=False, eos_token_id=None, pad_token_id=0)[0, len(ids):].tolist()
        want_text = hf.generate(input_ids=torch.tensor([text_only]), max_new_tokens=new, do_sample=False,
                                eos_token_id=None, pad_token_id=0)[0, len(text_only):].tolist()
    sp = SamplingParams(temperature=0.0, max_tokens=new, ignore_eos=True)
    seqs = eng.generate([ids, text_only], sp, mm_inputs=[{"pixel_values": px, "image_grid_thw": grid}, None])
    assert seqs[0].rope_delta == -8                    # 12 image tokens advance the position by max(3, 4)
    assert seqs[0].output == want, (seqs[0].output, want)
    assert seqs[1].output == want_text


def _hf3():
    from transformers import Qwen3VLConfig, Qwen3VLForConditionalGeneration
    torch.manual_seed(0)
    cfg = Qwen3VLConfig(
        text_config=dict(vocab_size=1024, hidden_size=128, intermediate_size=256, num_hidden_layers=3, num_attention_heads=4,
                         num_key_value_heads=2, head_dim=32, max_position_embeddings=512, rope_theta=10000.0,
                         rope_scaling={"rope_type": "default", "mrope_section": [4, 6, 6], "mrope_interleaved": True}),
        vision_config=dict(depth=3, hidden_size=64, intermediate_size=96, num_heads=4, patch_size=16, spatial_merge_size=2,
                           temporal_patch_size=2, out_hidden_size=128, num_position_embeddings=64, deepstack_visual_indexes=[0, 2]),
        image_token_id=1000, video_token_id=1001, vision_start_token_id=1002, vision_end_token_id=1003)
    m = Qwen3VLForConditionalGeneration(cfg).eval().float()
    for p in m.parameters():
        if p.dim() == 1:
            torch.nn.init.normal_(p, mean=0.5, std=0.2)
    return cfg, m


def test_qwen3_vl_tower_and_logits_match_hf():
    from chatlearn_b200.models.nn.model import packed_ctx
    from chatlearn_b200.models.nn.vision import VisionTower3
    from chatlearn_b200.models.nn.vl_model import VLCausalLM
    cfg, hf = _hf3()
    arch = _arch(cfg)
    assert arch.mrope_interleaved and arch.qk_norm and not arch.attention_bias
    model = VLCausalLM(arch)
    assert isinstance(model.visual, VisionTower3)
    model.load_hf_state_dict(hf.state_dict())
    grid = torch.tensor([[1, 6, 8], [1, 4, 4]])
    n = int((grid[:, 0] * grid[:, 1] * grid[:, 2]).sum())
    px = torch.randn(n, model.varch.patch_dim)
    with torch.no_grad():
        want_v = hf.model.visual(px, grid_thw=grid)
        got_v, taps = model.visual(px, grid)
    assert torch.allclose(got_v, want_v.pooler_output, rtol=1e-4, atol=1e-4)
    assert len(taps) == 2 and all(torch.allclose(a, b, rtol=1e-4, atol=1e-4) for a, b in zip(taps, want_v.deepstack_features))
    ids = torch.tensor([3, 4, 1002] + [1000] * 12 + [1003, 20, 21, 1002] + [1000] * 4 + [1003, 22, 23])
    with torch.no_grad():
        want = hf(input_ids=ids[None], pixel_values=px, image_grid_thw=grid, mm_token_type_ids=(ids[None] == 1000).long()).logits[0]
        ctx, _ = packed_ctx([ids.numel()], "cpu")
        ctx.mrope_positions = model.positions(ids, grid)
        got = model.logits(ids, ctx, px, grid)
    assert torch.allclose(got, want, rtol=3e-4, atol=3e-4), (got - want).abs().max()


def test_qwen3_vl_rollout_engine_generates_like_hf():
    from chatlearn_b200.models.nn.model import CausalLM
    from chatlearn_b200.models.nn.vision import build_vision_tower
    from chatlearn_b200.models.nn.vl_model import strip_language_prefix
    from chatlearn_b200.rollout import RolloutEngine, SamplingParams
    cfg, hf = _hf3()
    arch = _arch(cfg)
    arch.eos_token_id = 1023
    lm = CausalLM(arch)
    lm.load_hf_state_dict(strip_language_prefix(hf.state_dict()))
    tower = build_vision_tower(arch, torch.float32, "cpu")
    tower.load_hf_state_dict(hf.state_dict())
    eng = RolloutEngine(lm, block_size=8, num_blocks=64, max_num_seqs=4, max_num_batched_tokens=64, max_model_len=128,
                        vision=tower)
    grid = torch.tensor([[1, 6, 8]])
    ids = [3, 4, 1002] + [1000] * 12 + [1003, 20, 21, 22, 23]
    px = torch.randn(48, tower.arch.patch_dim)
    with torch.no_grad():
        want = hf.generate(input_ids=torch.tensor([ids]), pixel_values=px, image_grid_thw=grid,
                           mm_token_type_ids=(torch.tensor([ids]) == 1000).long(),
                           max_new_tokens=6, do_sample=False, eos_token_id=None, pad_token_id=0)[0, len(ids):].tolist()
    seqs = eng.generate([ids], SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True),
                        mm_inputs=[{"pixel_values": px, "image_grid_thw": grid}])
    assert seqs[0].output == want, (seqs[0].output, want)


def test_qwen3_vl_moe_logits_match_hf():
    """Qwen3-VL with a mixture-of-experts language model (the 30B-A3B vision-language checkpoints)."""
    from transformers import Qwen3VLMoeConfig, Qwen3VLMoeForConditionalGeneration
    from chatlearn_b200.models.nn.model import packed_ctx
    from chatlearn_b200.models.nn.vl_model import VLCausalLM
    torch.manual_seed(0)
    cfg = Qwen3VLMoeConfig(
        text_config=dict(vocab_size=1024, hidden_size=128, intermediate_size=256, num_hidden_layers=3, num_attention_heads=4,
                         num_key_value_heads=2, head_dim=32, max_position_embeddings=512, rope_theta=10000.0,
                         moe_intermediate_size=48, num_experts=8, num_experts_per_tok=2, decoder_sparse_step=1, mlp_only_layers=[],
                         norm_topk_prob=True,
                         rope_scaling={"rope_type": "default", "mrope_section": [4, 6, 6], "mrope_interleaved": True}),
        vision_config=dict(depth=3, hidden_size=64, intermediate_size=96, num_heads=4, patch_size=16, spatial_merge_size=2,
                           temporal_patch_size=2, out_hidden_size=128, num_position_embeddings=64, deepstack_visual_indexes=[0, 2]),
        image_token_id=1000, video_token_id=1001, vision_start_token_id=1002, vision_end_token_id=1003)
    hf = Qwen3VLMoeForConditionalGeneration(cfg).eval().float()
    for p in hf.parameters():
        if p.dim() == 1:
            torch.nn.init.normal_(p, mean=0.5, std=0.2)
        elif p.dim() == 3:                       # stacked expert weights are created uninitialised
            torch.nn.init.normal_(p, std=0.05)
    for n, p in hf.named_parameters():
        if n.endswith("mlp.gate.weight"):        # routers start at zero: every expert would tie
            torch.nn.init.normal_(p, std=0.5)
    arch = _arch(cfg)
    assert arch.is_moe and arch.num_experts == 8 and arch.mrope_interleaved
    sd = dict(hf.state_dict())
    for k in [k for k in sd if k.endswith("mlp.experts.gate_up_proj") or k.endswith("mlp.experts.down_proj")]:
        w = sd.pop(k)                            # checkpoints on disk hold one tensor per expert and projection
        pre = k.rsplit(".", 1)[0]
        for e in range(w.shape[0]):
            if k.endswith("gate_up_proj"):       # [experts, 2 * width, hidden]: gate rows, then up rows
                g, u = w[e].chunk(2, dim=0)
                sd[f"{pre}.{e}.gate_proj.weight"], sd[f"{pre}.{e}.up_proj.weight"] = g.contiguous(), u.contiguous()
            else:                                # [experts, hidden, width]
                sd[f"{pre}.{e}.down_proj.weight"] = w[e].contiguous()
    model = VLCausalLM(arch)
    model.load_hf_state_dict(sd)
    grid = torch.tensor([[1, 6, 8]])
    px = torch.randn(48, model.varch.patch_dim)
    ids = torch.tensor([3, 4, 1002] + [1000] * 12 + [1003, 20, 21, 22])
    with torch.no_grad():
        want = hf(input_ids=ids[None], pixel_values=px, image_grid_thw=grid, mm_token_type_ids=(ids[None] == 1000).long()).logits[0]
        ctx, _ = packed_ctx([ids.numel()], "cpu")
        ctx.mrope_positions = model.positions(ids, grid)
        got = model.logits(ids, ctx, px, grid)
    assert torch.allclose(got, want, rtol=3e-4, atol=3e-4), (got - want).abs().max()


def test_video_positions_follow_the_published_rule():
    """Qwen2.5-VL's documented example: a video of 3 temporal grid steps x 2 x 2 merged patches whose steps are 50
    temporal positions apart (2 s per step x 25 positions per second), followed by five text tokens."""
    from chatlearn_b200.models.nn.vision import mrope_positions
    ids = torch.tensor([1001] * 12 + [5, 6, 7, 8, 9])
    pos, delta = mrope_positions(ids, [[3, 4, 4]], 1000, 2, video_token_id=1001, time_steps=[2.0 * 25])
    assert pos[0].tolist() == [0] * 4 + [50] * 4 + [100] * 4 + [101, 102, 103, 104, 105]
    assert pos[1].tolist() == [0, 0, 1, 1] * 3 + [101, 102, 103, 104, 105]
    assert pos[2].tolist() == [0, 1, 0, 1] * 3 + [101, 102, 103, 104, 105]
    assert delta == 106 - 17
    # an image, text, then a video at half a second per step and 2 positions per second (one position per step)
    ids = torch.tensor([3, 1000, 1000, 1000, 1000, 4, 1001, 1001, 5])
    pos, _ = mrope_positions(ids, [[1, 4, 4], [2, 2, 2]], 1000, 2, video_token_id=1001, time_steps=[None, 1.0])
    assert pos[0].tolist() == [0, 1, 1, 1, 1, 3, 4, 5, 6] and pos[1].tolist() == [0, 1, 1, 2, 2, 3, 4, 4, 6]


def test_video_frames_become_patches_and_reach_the_model():
    """Frames -> temporal groups of two -> patches in the image order (checked against the image path on a video of
    one repeated frame), placeholder expansion in the order of the prompt, and a forward pass whose video rows take
    the tower's output (equal to HuggingFace's with the same positions)."""
    import numpy as np

    from chatlearn_b200.data.vision_utils import expand_image_tokens, image_to_patches, process_visuals, video_to_patches
    from chatlearn_b200.models.nn.model import packed_ctx
    from chatlearn_b200.models.nn.vl_model import VLCausalLM
    rng = np.random.default_rng(0)
    frame = lambda: rng.integers(0, 255, (56, 84, 3), dtype=np.uint8)          # noqa: E731
    f0 = frame()
    pv_img, g_img = image_to_patches(f0)
    pv_vid, g_vid, sec = video_to_patches([f0, f0, f0], fps=4.0)               # 3 frames: the last group is padded
    assert g_vid == (2, g_img[1], g_img[2]) and sec == 0.5
    n = pv_img.shape[0]
    assert torch.equal(pv_vid[:n], pv_img) and torch.equal(pv_vid[n:], pv_img)
    # order of the items follows the prompt: video placeholder first, then the image
    vid = [frame() for _ in range(4)]
    prompt = [7, 1002, 1001, 1003, 8, 1002, 1000, 1003, 9]
    pv, grids, steps = process_visuals(prompt, [f0], [{"frames": vid, "fps": 2.0}], 1000, 1001, tokens_per_second=2.0)
    assert grids == [[2, 4, 6], [1, 4, 6]] and steps == [2.0, None] and pv.shape[0] == 3 * 24
    ids = expand_image_tokens(prompt, grids, 1000, 2, 1001)
    assert ids.count(1001) == 12 and ids.count(1000) == 6 and ids.index(1001) < ids.index(1000)

    cfg, hf = _hf()
    model = VLCausalLM(_arch(cfg))
    assert model.arch.video_token_id == 1001
    model.load_hf_state_dict(hf.state_dict())
    t = torch.tensor(ids)
    pos = model.positions(t, grids, steps)
    nv = 2 * 24
    with torch.no_grad():
        # HuggingFace takes images and videos separately; its own position rule for videos differs between
        # releases, so both sides get the same positions
        want = hf(input_ids=t[None], pixel_values=pv[nv:], image_grid_thw=torch.tensor(grids[1:]),
                  pixel_values_videos=pv[:nv], video_grid_thw=torch.tensor(grids[:1]),
                  position_ids=pos[:, None, :]).logits[0]
        ctx, _ = packed_ctx([t.numel()], "cpu")
        ctx.mrope_positions = pos
        got = model.logits(t, ctx, pv, grids)
    assert torch.allclose(got, want, rtol=2e-4, atol=2e-4), (got - want).abs().max()


def test_rollout_engine_generates_with_a_video_prompt():
    """A record with a video and an image through the prompt pipeline into the rollout engine: greedy generation equals
    the argmax continuation of the full forward pass with the same positions (prefill in chunks of 16 tokens)."""
    import numpy as np

    from chatlearn_b200.data.prompt_dataset import VLPromptPipeline
    from chatlearn_b200.models.nn.model import CausalLM, packed_ctx
    from chatlearn_b200.models.nn.vision import VisionArch, VisionTower
    from chatlearn_b200.models.nn.vl_model import VLCausalLM, strip_language_prefix
    from chatlearn_b200.rollout import RolloutEngine, SamplingParams
    cfg, hf = _hf()
    arch = _arch(cfg)
    rng = np.random.default_rng(1)
    rec = {"input_ids": [7, 1002, 1001, 1003, 8, 1002, 1000, 1003, 9], "data_source": "x", "ground_truth": "",
           "images": [rng.integers(0, 255, (56, 56, 3), dtype=np.uint8)],
           "videos": [{"frames": [rng.integers(0, 255, (56, 84, 3), dtype=np.uint8) for _ in range(4)], "fps": 1.0}]}
    pipe = VLPromptPipeline([rec], 512, image_token_id=1000, video_token_id=1001, tokens_per_second=arch.tokens_per_second)
    s = pipe.data[0]
    assert s["image_grid_thw"] == [[2, 4, 6], [1, 4, 4]] and s["visual_time_steps"] == [2.0, None]
    ids = s["input_ids"]
    assert len(ids) == 7 + 12 + 4 and s["prompt_token_length"] == len(ids)

    full = VLCausalLM(arch)
    full.load_hf_state_dict(hf.state_dict())
    new, cur = 6, list(ids)
    for _ in range(new):                                   # reference: one full forward per generated token
        t = torch.tensor(cur)
        ctx, _ = packed_ctx([t.numel()], "cpu")
        ctx.mrope_positions = full.positions(t, s["image_grid_thw"], s["visual_time_steps"])
        with torch.no_grad():
            cur.append(int(full.logits(t, ctx, s["pixel_values"], s["image_grid_thw"])[-1].argmax()))
    lm = CausalLM(arch)
    lm.load_hf_state_dict(strip_language_prefix(hf.state_dict()))
    tower = VisionTower(VisionArch.from_hf_dict(cfg.vision_config.to_dict()))
    tower.load_hf_state_dict(hf.state_dict())
    eng = RolloutEngine(lm, block_size=8, num_blocks=64, max_num_seqs=4, max_num_batched_tokens=16, max_model_len=128,
                        vision=tower)
    mm = {k: s[k] for k in ("pixel_values", "image_grid_thw", "visual_time_steps")}
    out = eng.generate([ids], SamplingParams(temperature=0.0, max_tokens=new, ignore_eos=True), mm_inputs=[mm])
    assert out[0].output == cur[len(ids):], (out[0].output, cur[len(ids):])


def test_placeholder_tokens_in_a_response_are_text():
    """A response may contain the image placeholder id (sampled like any token): positions and image rows follow
    the prompt's images only."""
    from chatlearn_b200.models.nn.vision import mrope_positions
    ids = torch.tensor([5, 1000, 1000, 1000, 1000, 6, 7, 1000, 8, 1001, 1001, 9])
    pos, delta = mrope_positions(ids, [[1, 4, 4]], 1000, 2, video_token_id=1001)
    assert pos[0].tolist() == [0, 1, 1, 1, 1, 3, 4, 5, 6, 7, 8, 9] and pos[2].tolist() == [0, 1, 2, 1, 2, 3, 4, 5, 6, 7, 8, 9]
    assert delta == 10 - 12


def test_video_file_is_decoded_and_sampled(tmp_path):
    """A 12-frame clip at 8 frames per second sampled at 2 per second gives 3 frames (the first of every 4), and goes
    through the prompt pipeline's item list like decoded frames do."""
    cv2 = pytest.importorskip("cv2")
    import numpy as np

    from chatlearn_b200.data.vision_utils import load_video, process_visuals
    path = str(tmp_path / "clip.avi")
    wr = cv2.VideoWriter(path, cv2.VideoWriter_fourcc(*"MJPG"), 8.0, (84, 56))
    if not wr.isOpened():
        pytest.skip("this OpenCV build cannot write MJPG")
    for i in range(12):
        wr.write(np.full((56, 84, 3), 20 * i, dtype=np.uint8))
    wr.release()
    frames, rate = load_video(path, fps=2.0)
    assert len(frames) == 3 and abs(rate - 2.0) < 1e-6 and frames[0].shape == (56, 84, 3)
    levels = [int(f.mean()) for f in frames]
    assert abs(levels[0] - 0) <= 3 and abs(levels[1] - 80) <= 3 and abs(levels[2] - 160) <= 3
    pv, grids, steps = process_visuals([7, 1001, 8], [], [{"path": path, "fps": 2.0}], 1000, 1001, tokens_per_second=2.0)
    assert grids == [[2, 4, 6]] and steps == [2.0] and pv.shape[0] == 48
