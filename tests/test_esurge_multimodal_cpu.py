"""Images through the serving engine on CPU: resolution buckets, feature cache, placeholder expansion, chunked
prefill across an image, and engine output equal to the model's own greedy decoding."""

import numpy as np
import torch

from easydel_b200.inference import SamplingParams
from easydel_b200.inference.esurge import eSurge
from easydel_b200.inference.esurge.multimodal import MultiModalManager, VisionEncoderCache
from easydel_b200.modules.llava import LlavaConfig, LlavaForConditionalGeneration

IMG = 127


def _model():
    torch.manual_seed(0)
    cfg = LlavaConfig(
        vision_config=dict(model_type="clip_vision_model", hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                           num_attention_heads=4, image_size=28, patch_size=14),
        text_config=dict(model_type="llama", vocab_size=128, hidden_size=32, intermediate_size=64,
                         num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                         max_position_embeddings=512, eos_token_id=126),
        image_token_index=IMG, vision_feature_layer=-1)
    return LlavaForConditionalGeneration(cfg, dtype=torch.float32, param_dtype=torch.float32).eval()


def _image(seed, size=(40, 30)):
    return (np.random.default_rng(seed).random((size[1], size[0], 3)) * 255).astype(np.uint8)


def test_feature_cache_lru_and_budget():
    c = VisionEncoderCache(capacity_mb=1)
    a = torch.zeros(64, 1024)            # 256 KiB each
    for i in range(5):
        c.put(f"k{i}", a + i)
    assert len(c) == 4 and not c.contains("k0") and c.size_mb <= 1.0
    assert c.get("k1") is not None and c.get("k0") is None
    c.put("k5", a)                       # k2 is now the oldest
    assert not c.contains("k2") and c.contains("k1")
    assert c.get_stats()["hits"] == 1 and c.get_stats()["misses"] == 1
    c.put("huge", torch.zeros(1024, 1024))
    assert not c.contains("huge")


def test_manager_buckets_placeholders_and_cache():
    m = _model()
    mgr = MultiModalManager(m)
    px = mgr.process_images([_image(0), _image(1, (28, 28))])
    assert all(p.shape == (3, 28, 28) for p in px)
    ids, embeds, key = mgr.prepare([5, IMG, 6, IMG, 7], [_image(0), _image(1)])
    rows = embeds[0][1].shape[0]
    assert rows == 4 and ids == [5] + [IMG] * 4 + [6] + [IMG] * 4 + [7]
    assert [o for o, _ in embeds] == [1, 6] and len(set(key)) == 2
    before = mgr.get_cache_stats()["misses"]
    ids2, embeds2, key2 = mgr.prepare([IMG] * 4 + [9], [_image(0)])     # an already expanded run, a cached image
    assert ids2 == [IMG] * 4 + [9] and key2[0] == key[0]
    assert mgr.get_cache_stats()["misses"] == before and torch.equal(embeds2[0][1], embeds[0][1])
    msgs = [{"role": "user", "content": [{"type": "text", "text": "look: "},
                                          {"type": "image_url", "image_url": {"url": "data:image/png;base64,AAAA"}},
                                          {"type": "image", "image": _image(3)}]}]
    images, videos = mgr.extract_media_from_messages(msgs)
    assert len(images) == 2 and not videos and images[0].startswith("data:")
    assert mgr.normalize_messages(msgs, "<image>")[0]["content"] == "look: <image><image>"


def _greedy(m, ids, images, n, mgr):
    full_ids, embeds, _ = mgr.prepare(ids, images)
    toks = list(full_ids)
    for _ in range(n):
        t = torch.tensor([toks])
        emb = m.get_input_embeddings()(t)
        for off, f in embeds:
            emb[0, off:off + f.shape[0]] = f
        with torch.no_grad():
            nxt = int(m.language_model(inputs_embeds=emb).logits[0, -1].argmax())
        toks.append(nxt)
    return toks[len(full_ids):]


def test_engine_serves_images_like_the_model_even_across_prefill_chunks():
    m = _model()
    prompt = [3, 4, IMG, 9, 10, 11, IMG, 12]
    imgs = [_image(0), _image(1)]
    for budget in (64, 5):       # 5 tokens per step: both images are split across engine steps
        eng = eSurge(m, max_model_len=256, max_num_seqs=2, max_num_batched_tokens=budget, num_pages=8)
        want = _greedy(m, prompt, imgs, 6, eng.multimodal)
        out = eng.generate(prompt, SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True), images=imgs)[0]
        assert list(out.outputs[0].token_ids) == want, (budget, out.outputs[0].token_ids, want)
    # other images behind the same tokens do not hit the prefix cache of the first request
    other = eng.generate(prompt, SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True),
                         images=[_image(5), _image(6)])[0]
    assert list(other.outputs[0].token_ids) == _greedy(m, prompt, [_image(5), _image(6)], 6, eng.multimodal)


def test_flat_patch_tower_images_and_videos_expand_in_one_pass():
    """Qwen-VL style towers: the manager cuts frames into merge-block-ordered patch rows with a (t, h, w) grid; image
    and video placeholders are expanded together and the rows equal a direct call of the tower."""
    import numpy as np

    from easydel_b200.modules.qwen2_vl import Qwen2VLConfig, Qwen2VLForConditionalGeneration

    V = dict(depth=1, embed_dim=32, hidden_size=32, num_heads=4, in_channels=3, patch_size=4, spatial_merge_size=2,
             temporal_patch_size=2, mlp_ratio=2)
    T = dict(vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=4,
             num_key_value_heads=2, rope_scaling={"type": "mrope", "mrope_section": [1, 1, 2]})
    torch.manual_seed(0)
    model = Qwen2VLForConditionalGeneration(Qwen2VLConfig(vision_config=V, text_config=T, image_token_id=127,
                                                          video_token_id=126), dtype=torch.float32).eval()
    mgr = MultiModalManager(model, resolution_buckets=[(16, 16)])
    assert mgr.flat_patch
    rng = np.random.default_rng(0)
    image = rng.integers(0, 255, (16, 16, 3), dtype=np.uint8)
    video = rng.integers(0, 255, (3, 16, 16, 3), dtype=np.uint8)      # 3 frames -> 2 temporal patches
    ids, embeds, key = mgr.prepare([5, 126, 6, 127, 7], images=[image], videos=[video])
    assert ids == [5] + [126] * 8 + [6] + [127] * 4 + [7]
    assert [o for o, _ in embeds] == [1, 10] and [e.shape for _, e in embeds] == [(8, 32), (4, 32)]
    frames = torch.stack(mgr.process_images(list(video)))
    rows, grid = mgr.patchify(frames)
    assert grid == (2, 4, 4) and rows.shape == (32, 3 * 2 * 16)
    # block order: the first four rows are the 2 x 2 merge block at the top-left of the first temporal patch
    want = torch.stack([frames[0:2, :, 0:4, 0:4], frames[0:2, :, 0:4, 4:8], frames[0:2, :, 4:8, 0:4],
                        frames[0:2, :, 4:8, 4:8]]).permute(0, 2, 1, 3, 4).reshape(4, -1)
    torch.testing.assert_close(rows[:4], want)
    with torch.no_grad():
        direct = model.get_video_features(rows, video_grid_thw=torch.tensor([grid]))
    torch.testing.assert_close(embeds[0][1], direct)
    assert len(key) == 2


def test_three_stream_rotary_positions_through_the_engine():
    """Qwen2-VL style rotary: vision tokens sit at (temporal, row, column) coordinates and the text after them
    continues from the largest. The manager computes the same positions as the model's own routine, the runner
    stages them beside the token indices (chunked prefill across the vision runs included), and the engine's greedy
    tokens equal a plain forward loop of the model that is handed those positions."""
    from easydel_b200.modules.qwen2_vl import Qwen2VLConfig, Qwen2VLForConditionalGeneration, mrope_positions

    V = dict(depth=1, embed_dim=32, hidden_size=32, num_heads=4, in_channels=3, patch_size=4, spatial_merge_size=2,
             temporal_patch_size=2, mlp_ratio=2)
    T = dict(vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
             num_key_value_heads=2, max_position_embeddings=512, eos_token_id=125,
             rope_scaling={"type": "mrope", "mrope_section": [2, 1, 1]})
    NTOK = 24
    torch.manual_seed(0)
    model = Qwen2VLForConditionalGeneration(Qwen2VLConfig(vision_config=V, text_config=T, image_token_id=127,
                                                          video_token_id=126), dtype=torch.float32).eval()
    rng = np.random.default_rng(1)
    image = rng.integers(0, 255, (16, 24, 3), dtype=np.uint8)
    video = rng.integers(0, 255, (4, 16, 16, 3), dtype=np.uint8)
    prompt = [5, 9, 126, 6, 11, 127, 7, 8]
    eng = eSurge(model, max_model_len=256, max_num_seqs=2, max_num_batched_tokens=8, hbm_utilization=0.05,
                 enable_prefix_caching=False)
    try:
        mgr = eng.multimodal
        mgr.resolution_buckets = [(16, 16), (24, 16)]
        ids, embeds, _, rope = mgr.prepare(prompt, images=[image], videos=[video], with_rope=True)
        assert rope is not None
        pos, delta = rope
        # the model's own routine on the expanded ids and the grids of the two runs
        grids = {o: None for o, _ in embeds}
        _, vg = mgr.patchify(torch.stack(mgr.process_images(list(video))))
        _, ig = mgr.patchify(mgr.process_images([image])[0][None])
        vid_grid, img_grid = torch.tensor([list(vg)]), torch.tensor([list(ig)])
        assert vg[0] == 2 and ig[0] == 1
        want, want_delta = mrope_positions(torch.tensor([ids]), 127, img_grid, 2, video_token_id=126,
                                           video_grid_thw=vid_grid)
        assert np.array_equal(pos, want[:, 0].numpy()) and delta == int(want_delta[0])
        assert delta < 0 and len(grids) == 2          # vision runs advance the position by less than their length
        out = eng.generate(prompt, SamplingParams(max_tokens=NTOK, temperature=0.0, ignore_eos=True), images=[image],
                           videos=[video])[0]
        got = list(out.outputs[0].token_ids)
    finally:
        eng.close()
    # reference: full forward passes of the language model on the spliced embeddings with those positions
    lm = model.language_model
    toks = list(ids)
    ref = []
    with torch.no_grad():
        for _ in range(NTOK):
            n = len(toks)
            emb = lm.get_input_embeddings()(torch.tensor([toks]))
            for off, feats in embeds:
                emb[0, off:off + feats.shape[0]] = feats
            p = torch.zeros(3, 1, n, dtype=torch.long)
            p[:, 0, :len(ids)] = torch.from_numpy(pos).long()
            if n > len(ids):
                p[:, 0, len(ids):] = torch.arange(len(ids), n) + delta
            logits = lm(inputs_embeds=emb, position_ids=p).logits
            nxt = int(logits[0, -1].argmax())
            ref.append(nxt)
            toks.append(nxt)
    assert got == ref
    # the positions matter to this model: consecutive numbering changes the logits of the first generated token
    with torch.no_grad():
        emb = lm.get_input_embeddings()(torch.tensor([ids]))
        for off, feats in embeds:
            emb[0, off:off + feats.shape[0]] = feats
        a = lm(inputs_embeds=emb, position_ids=torch.from_numpy(pos).long()[:, None]).logits[0, -1]
        b = lm(inputs_embeds=emb, position_ids=torch.arange(len(ids))[None]).logits[0, -1]
    assert (a - b).abs().max() > 1e-4
