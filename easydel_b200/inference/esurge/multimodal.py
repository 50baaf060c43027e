"""Images in the serving engine (easydel/inference/esurge/multimodal/{manager,cache,types}.py).

* :class:`MultiModalManager` turns the images of a request (PIL images, arrays, paths, ``data:`` URLs inside OpenAI
  chat messages) into normalised pixel tensors at one of a few fixed resolutions (so the vision tower only ever sees
  a handful of shapes), runs the model's vision tower + projector once per distinct image, and rewrites the prompt so
  that every image placeholder token is repeated once per image feature row.
* :class:`VisionEncoderCache` keeps projected image features on the device under a byte budget, keyed by a hash of
  the pixels: a repeated image (multi-turn chat, shared system image) costs no tower forward.
* The engine stores ``(offset, features)`` on the request; the runner embeds the step's tokens and overwrites the
  placeholder rows that fall inside the scheduled range (chunked prefill splits an image across steps without any
  special handling). The feature hashes join the page hashes so that prefix caching never matches two prompts that
  differ only in their images.
"""

from __future__ import annotations

import base64
import hashlib
import io
import typing as tp
from collections import OrderedDict
from dataclasses import dataclass, field

import numpy as np
import torch

CLIP_MEAN, CLIP_STD = (0.48145466, 0.4578275, 0.40821073), (0.26862954, 0.26130258, 0.27577711)
HALF_MEAN, HALF_STD = (0.5, 0.5, 0.5), (0.5, 0.5, 0.5)


@dataclass
class PlaceholderRange:
    offset: int
    length: int

    @property
    def end(self) -> int:
        return self.offset + self.length


@dataclass
class MultiModalFeature:
    mm_hash: str
    modality: str = "image"
    pixel_values: torch.Tensor | None = None           # [3, H, W], dropped once the embeddings exist
    embeddings: torch.Tensor | None = None             # [rows, hidden] on the model's device
    placeholder: PlaceholderRange | None = None
    grid: tuple | None = None                          # (t, h, w) in patches, towers that take flattened patches

    @classmethod
    def from_image(cls, pixel_values: torch.Tensor) -> "MultiModalFeature":
        return cls(mm_hash=hash_pixels(pixel_values), pixel_values=pixel_values)

    @property
    def has_cached_embeddings(self) -> bool:
        return self.embeddings is not None

    def clear_pixel_values(self) -> None:
        self.pixel_values = None


@dataclass
class BatchedMultiModalInputs:
    """Images of several requests stacked for one tower forward."""

    pixel_values: torch.Tensor | None = None
    request_index: list[int] = field(default_factory=list)

    @classmethod
    def from_features(cls, per_request: list[list[MultiModalFeature]]) -> "BatchedMultiModalInputs":
        px, idx = [], []
        for r, feats in enumerate(per_request):
            for f in feats:
                if f.pixel_values is not None:
                    px.append(f.pixel_values)
                    idx.append(r)
        return cls(torch.stack(px) if px else None, idx)

    @property
    def has_images(self) -> bool:
        return self.pixel_values is not None

    @property
    def num_images(self) -> int:
        return len(self.request_index)

    def get_request_image_count(self, request_idx: int) -> int:
        return sum(1 for r in self.request_index if r == request_idx)


def hash_pixels(pixel_values: torch.Tensor | np.ndarray) -> str:
    a = pixel_values.detach().cpu().contiguous().numpy() if isinstance(pixel_values, torch.Tensor) else \
        np.ascontiguousarray(pixel_values)
    h = hashlib.blake2b(digest_size=16)
    h.update(str(a.shape).encode())
    h.update(str(a.dtype).encode())
    h.update(a.tobytes())
    return h.hexdigest()


class VisionEncoderCache:
    """LRU over projected image features with a byte budget."""

    def __init__(self, capacity_mb: int = 1024):
        self.capacity = int(capacity_mb) << 20
        self._items: OrderedDict[str, torch.Tensor] = OrderedDict()
        self._bytes = 0
        self.hits = self.misses = 0

    compute_hash = staticmethod(hash_pixels)

    def get(self, key: str) -> torch.Tensor | None:
        t = self._items.get(key)
        if t is None:
            self.misses += 1
            return None
        self._items.move_to_end(key)
        self.hits += 1
        return t

    def put(self, key: str, embeddings: torch.Tensor) -> None:
        n = embeddings.numel() * embeddings.element_size()
        if n > self.capacity:
            return
        old = self._items.pop(key, None)
        if old is not None:
            self._bytes -= old.numel() * old.element_size()
        while self._items and self._bytes + n > self.capacity:
            _, ev = self._items.popitem(last=False)
            self._bytes -= ev.numel() * ev.element_size()
        self._items[key] = embeddings
        self._bytes += n

    def contains(self, key: str) -> bool:
        return key in self._items

    def clear(self) -> None:
        self._items.clear()
        self._bytes = 0

    def __len__(self) -> int:
        return len(self._items)

    @property
    def size_mb(self) -> float:
        return self._bytes / (1 << 20)

    @property
    def hit_rate(self) -> float:
        n = self.hits + self.misses
        return self.hits / n if n else 0.0

    def get_stats(self) -> dict:
        return {"entries": len(self), "size_mb": self.size_mb, "capacity_mb": self.capacity / (1 << 20),
                "hits": self.hits, "misses": self.misses, "hit_rate": self.hit_rate}


class MultiModalManager:
    def __init__(self, model, tokenizer=None, processor=None, resolution_buckets: list[tuple[int, int]] | None = None,
                 cache_capacity_mb: int = 1024, enable_cache: bool = True, max_batch_images: int = 16):
        self.model, self.tokenizer, self.processor = model, tokenizer, processor
        self.cache = VisionEncoderCache(cache_capacity_mb) if enable_cache else None
        self.max_batch_images = max_batch_images
        cfg = model.config
        self.vision_config = getattr(cfg, "vision_config", None)
        self.image_token_id = getattr(cfg, "image_token_index", getattr(cfg, "image_token_id", None))
        size = getattr(self.vision_config, "image_size", 224)
        # fixed-size towers accept exactly one resolution; others snap to the closest bucket
        self.buckets = resolution_buckets or [(size, size)]
        vt = getattr(self.vision_config, "model_type", "")
        self.mean, self.std = (HALF_MEAN, HALF_STD) if "siglip" in vt else (CLIP_MEAN, CLIP_STD)
        ip = getattr(processor, "image_processor", None)
        if ip is not None and getattr(ip, "image_mean", None) is not None:
            self.mean, self.std = tuple(ip.image_mean), tuple(ip.image_std)
        self.video_token_id = getattr(cfg, "video_token_id", None)
        # towers that take flattened [temporal x patch x patch] pixel blocks plus a (t, h, w) grid per item
        vc = self.vision_config
        self.flat_patch = all(hasattr(vc, k) for k in ("spatial_merge_size", "temporal_patch_size", "patch_size"))
        if self.flat_patch and resolution_buckets is None:
            unit = vc.patch_size * vc.spatial_merge_size
            self.buckets = [(unit * a, unit * b) for a, b in ((8, 8), (12, 8), (8, 12), (16, 16), (24, 16), (16, 24))]

    # ------------------------------------------------------------------ pixels
    def resize_to_bucket(self, image):
        from PIL import Image

        w, h = image.size
        ar = w / max(h, 1)
        bw, bh = min(self.buckets, key=lambda b: (abs(b[0] / b[1] - ar), abs(b[0] * b[1] - w * h)))
        if (w, h) == (bw, bh):
            return image
        return image.resize((bw, bh), Image.BICUBIC)

    def _to_pil(self, img):
        from PIL import Image

        if isinstance(img, Image.Image):
            return img.convert("RGB")
        if isinstance(img, (bytes, bytearray)):
            return Image.open(io.BytesIO(bytes(img))).convert("RGB")
        if isinstance(img, str):
            if img.startswith("data:"):
                return Image.open(io.BytesIO(base64.b64decode(img.split(",", 1)[1]))).convert("RGB")
            if img.startswith(("http://", "https://")):
                import requests

                return Image.open(io.BytesIO(requests.get(img, timeout=30).content)).convert("RGB")
            return Image.open(img).convert("RGB")
        if isinstance(img, torch.Tensor):
            img = img.detach().cpu().numpy()
        a = np.asarray(img)
        if a.ndim == 3 and a.shape[0] in (1, 3) and a.shape[-1] not in (1, 3):
            a = a.transpose(1, 2, 0)
        if a.dtype != np.uint8:
            a = (np.clip(a, 0.0, 1.0) * 255).astype(np.uint8) if a.max() <= 1.0 else a.astype(np.uint8)
        return Image.fromarray(a).convert("RGB")

    def _normalize_rgb(self, rgb: np.ndarray) -> np.ndarray:
        x = rgb.astype(np.float32) / 255.0
        return (x - np.asarray(self.mean, np.float32)) / np.asarray(self.std, np.float32)

    def process_images(self, images: tp.Sequence[tp.Any]) -> list[torch.Tensor]:
        """-> one ``[3, H, W]`` fp32 tensor per image (resolutions may differ across buckets)."""
        out = []
        for img in images:
            pil = self.resize_to_bucket(self._to_pil(img))
            out.append(torch.from_numpy(self._normalize_rgb(np.asarray(pil)).transpose(2, 0, 1).copy()))
        return out

    def patchify(self, frames: torch.Tensor) -> tuple[torch.Tensor, tuple[int, int, int]]:
        """``[T, 3, H, W]`` normalised frames -> (``[t * h * w, 3 * tp * P * P]`` rows ordered merge block by merge
        block, ``(t, h, w)`` grid in patches). A frame count that is not a multiple of the temporal patch repeats the
        last frame (a still image is one temporal patch of identical frames)."""
        vc = self.vision_config
        P, tp, m = vc.patch_size, vc.temporal_patch_size, vc.spatial_merge_size
        T, C, H, W = frames.shape
        if T % tp:
            frames = torch.cat([frames, frames[-1:].expand(tp - T % tp, C, H, W)])
        gt, gh, gw = frames.shape[0] // tp, H // P, W // P
        if H % (P * m) or W % (P * m):
            raise ValueError(f"frame size {H}x{W} is not a multiple of patch {P} x merge {m}")
        x = frames.reshape(gt, tp, C, gh // m, m, P, gw // m, m, P)
        x = x.permute(0, 3, 6, 4, 7, 2, 1, 5, 8).reshape(gt * gh * gw, C * tp * P * P)
        return x.contiguous(), (gt, gh, gw)

    def process_videos(self, videos: tp.Sequence[tp.Any], max_frames: int = 32) -> list[torch.Tensor]:
        """Each video (``[T, H, W, 3]`` / ``[T, 3, H, W]`` array, or a list of frames) -> ``[T', 3, H, W]`` fp32:
        at most ``max_frames`` frames sampled uniformly, all resized to one resolution bucket."""
        out = []
        for v in videos:
            if isinstance(v, torch.Tensor):
                v = v.detach().cpu().numpy()
            frames = list(v) if not isinstance(v, (list, tuple)) else list(v)
            if len(frames) > max_frames:
                idx = np.linspace(0, len(frames) - 1, max_frames).round().astype(int)
                frames = [frames[i] for i in idx]
            out.append(torch.stack(self.process_images(frames)))
        return out

    # ------------------------------------------------------------------ messages
    @staticmethod
    def extract_media_from_messages(messages: list[dict]) -> tuple[list[tp.Any], list[tp.Any]]:
        """OpenAI-style content parts -> (images, videos) in order of appearance."""
        images, videos = [], []
        for m in messages:
            content = m.get("content")
            if not isinstance(content, list):
                continue
            for part in content:
                if not isinstance(part, dict):
                    continue
                kind = part.get("type")
                if kind in ("image", "input_image"):
                    src = part.get("image", part.get("url", part.get("image_url")))
                    if src is not None:
                        images.append(src["url"] if isinstance(src, dict) else src)
                elif kind == "image_url":
                    src = part.get("image_url")
                    images.append(src["url"] if isinstance(src, dict) else src)
                elif kind in ("video", "video_url"):
                    src = part.get("video", part.get("video_url"))
                    videos.append(src["url"] if isinstance(src, dict) else src)
        return images, videos

    def normalize_messages(self, messages: list[dict], placeholder: str | None = None) -> list[dict]:
        """Flattens content parts to text for chat templates that know nothing about images: every image part
        becomes the placeholder token's text."""
        ph = placeholder or self._placeholder_text() or "<image>"
        out = []
        for m in messages:
            content = m.get("content")
            if isinstance(content, list):
                text = "".join(ph if (isinstance(p, dict) and p.get("type") in ("image", "image_url", "input_image"))
                               else (p.get("text", "") if isinstance(p, dict) else str(p)) for p in content)
                m = dict(m, content=text)
            out.append(m)
        return out

    def _placeholder_text(self) -> str | None:
        if self.tokenizer is None or self.image_token_id is None:
            return None
        try:
            return self.tokenizer.convert_ids_to_tokens(int(self.image_token_id))
        except Exception:
            return None

    # ------------------------------------------------------------------ features
    @torch.no_grad()
    def process_images_to_features(self, images: tp.Sequence[tp.Any]) -> list[MultiModalFeature]:
        feats = [MultiModalFeature.from_image(p) for p in self.process_images(images)]
        todo: dict[str, MultiModalFeature] = {}
        for f in feats:
            hit = self.cache.get(f.mm_hash) if self.cache is not None else None
            if hit is not None:
                f.embeddings = hit
            else:
                todo.setdefault(f.mm_hash, f)
        dev = next(self.model.parameters()).device
        pending = list(todo.values())
        if self.flat_patch:
            for f in pending:
                self._encode_flat(f, dev)
            pending = []
        # one tower forward per resolution bucket and chunk of images
        by_shape: dict[tuple, list[MultiModalFeature]] = {}
        for f in pending:
            by_shape.setdefault(tuple(f.pixel_values.shape), []).append(f)
        for group in by_shape.values():
            for i in range(0, len(group), self.max_batch_images):
                chunk = group[i:i + self.max_batch_images]
                px = torch.stack([f.pixel_values for f in chunk]).to(dev, self.model.dtype)
                emb = self.model.get_image_features(px)
                emb = emb.reshape(len(chunk), -1, emb.shape[-1])
                for f, e in zip(chunk, emb):
                    f.embeddings = e.contiguous()
                    if self.cache is not None:
                        self.cache.put(f.mm_hash, f.embeddings)
        for f in feats:
            if f.embeddings is None:
                f.embeddings = todo[f.mm_hash].embeddings
            self.grid_of(f)
            f.clear_pixel_values()
        return feats

    def _encode_flat(self, f: MultiModalFeature, dev) -> None:
        frames = f.pixel_values if f.pixel_values.dim() == 4 else f.pixel_values[None]
        rows, grid = self.patchify(frames)
        f.grid = tuple(int(g) for g in grid)
        grid_t = torch.tensor([grid], device=dev)
        fn = self.model.get_video_features if (f.modality == "video" and hasattr(self.model, "get_video_features")) \
            else self.model.get_image_features
        key = "video_grid_thw" if fn.__name__ == "get_video_features" else "image_grid_thw"
        f.embeddings = fn(rows.to(dev, self.model.dtype), **{key: grid_t}).contiguous()
        if self.cache is not None:
            self.cache.put(f.mm_hash, f.embeddings)

    @torch.no_grad()
    def process_videos_to_features(self, videos: tp.Sequence[tp.Any]) -> list[MultiModalFeature]:
        if not self.flat_patch:
            raise ValueError("this model's vision tower takes single images; pass the frames as images")
        dev = next(self.model.parameters()).device
        feats = []
        for frames in self.process_videos(videos):
            f = MultiModalFeature(mm_hash=hash_pixels(frames), modality="video", pixel_values=frames)
            hit = self.cache.get(f.mm_hash) if self.cache is not None else None
            if hit is not None:
                f.embeddings = hit
            else:
                self._encode_flat(f, dev)
            self.grid_of(f)
            f.clear_pixel_values()
            feats.append(f)
        return feats

    def expand_placeholders(self, token_ids: tp.Sequence[int], feats: list[MultiModalFeature],
                            placeholder_id: int | None = None) -> list[int]:
        """Repeats the i-th placeholder once per row of the i-th feature and records where it landed.
        A run of placeholders already as long as the feature (a processor expanded it) is left as it is."""
        ph = self.image_token_id if placeholder_id is None else placeholder_id
        return self._expand(token_ids, {ph: feats})

    @staticmethod
    def _expand(token_ids: tp.Sequence[int], by_token: dict[int, list[MultiModalFeature]]) -> list[int]:
        out: list[int] = []
        used = {ph: 0 for ph in by_token}
        i, n = 0, len(token_ids)
        while i < n:
            t = token_ids[i]
            if t not in by_token:
                out.append(t)
                i += 1
                continue
            feats = by_token[t]
            j = i
            while j < n and token_ids[j] == t:
                j += 1
            run = j - i
            while run > 0:
                k = used[t]
                if k >= len(feats):
                    raise ValueError("more media placeholders in the prompt than media items in the request")
                rows = feats[k].embeddings.shape[0]
                take = rows if run >= rows else 1
                feats[k].placeholder = PlaceholderRange(len(out), rows)
                out.extend([t] * rows)
                run -= take
                used[t] = k + 1
            i = j
        for ph, feats in by_token.items():
            if used[ph] != len(feats):
                raise ValueError(f"{len(feats)} media items for {used[ph]} placeholders of token {ph} in the prompt")
        return out

    def grid_of(self, f: MultiModalFeature) -> tuple | None:
        """(t, h, w) patch grid of a feature of a flattened-patch tower (kept on the feature; recomputed from the
        number of rows and the frame shape when the embeddings came from the cache)."""
        if f.grid is None and self.flat_patch and f.pixel_values is not None:
            frames = f.pixel_values if f.pixel_values.dim() == 4 else f.pixel_values[None]
            vc = self.model.config.vision_config
            t = -(-frames.shape[0] // vc.temporal_patch_size)
            f.grid = (int(t), int(frames.shape[-2] // vc.patch_size), int(frames.shape[-1] // vc.patch_size))
        return f.grid

    def rope_positions(self, num_tokens: int, feats: tp.Sequence[MultiModalFeature]):
        """Three-stream rotary positions of a prompt whose vision placeholders are ``feats``: text advances all three
        streams together, a vision run takes (temporal, row, column) indices from where the text stopped and the
        text after it continues from the largest of them (the arithmetic of ``mrope_positions`` in
        ``modules/qwen2_vl``). -> (``[3, num_tokens]`` int32, offset of generated tokens from their index)."""
        import numpy as np

        m = int(self.model.config.vision_config.spatial_merge_size)
        pos = np.zeros((3, num_tokens), dtype=np.int32)
        cur, i = 0, 0
        for f in sorted(feats, key=lambda f: f.placeholder.offset):
            a = f.placeholder.offset
            if a > i:
                pos[:, i:a] = cur + np.arange(a - i, dtype=np.int32)
                cur += a - i
            t, h, w = f.grid
            gh, gw = h // m, w // m
            n = t * gh * gw
            if n != f.placeholder.length:
                raise ValueError(f"vision run of {f.placeholder.length} tokens does not match its grid {f.grid}")
            ti, hi, wi = np.meshgrid(np.arange(t), np.arange(gh), np.arange(gw), indexing="ij")
            pos[:, a:a + n] = cur + np.stack([ti.reshape(-1), hi.reshape(-1), wi.reshape(-1)]).astype(np.int32)
            cur += max(t, gh, gw)
            i = a + n
        if i < num_tokens:
            pos[:, i:] = cur + np.arange(num_tokens - i, dtype=np.int32)
            cur += num_tokens - i
        return pos, int(cur - num_tokens)

    @property
    def three_stream_rotary(self) -> bool:
        """Whether the language model rotates with three position streams (vision tokens at grid coordinates)."""
        cfg = getattr(self.model.config, "text_config", None) or self.model.config
        rs = getattr(cfg, "rope_scaling", None) or getattr(self.model.config, "rope_scaling", None) or {}
        return self.flat_patch and isinstance(rs, dict) and "mrope_section" in rs

    def prepare(self, token_ids: tp.Sequence[int], images: tp.Sequence[tp.Any] | None = None,
                videos: tp.Sequence[tp.Any] | None = None, with_rope: bool = False):
        """-> (expanded token ids, [(offset, embeddings)], extra hash key) for ``eSurge.add_request``; with
        ``with_rope`` a fourth item: ``(positions [3, tokens], delta)`` for three-stream rotary models (None for
        the others), so that the engine rotates vision tokens at their grid coordinates as ``model.generate`` does."""
        feats = self.process_images_to_features(images) if images else []
        vfeats = self.process_videos_to_features(videos) if videos else []
        by_token = {}
        want_rope = with_rope and self.three_stream_rotary
        if feats:
            by_token[self.image_token_id] = feats
        if vfeats:
            by_token[self.video_token_id] = vfeats
        ids = self._expand(list(token_ids), by_token) if by_token else list(token_ids)
        allf = sorted(feats + vfeats, key=lambda f: f.placeholder.offset)
        out = (ids, [(f.placeholder.offset, f.embeddings) for f in allf], tuple(f.mm_hash for f in allf))
        if not with_rope:
            return out
        rope = self.rope_positions(len(ids), allf) if want_rope and all(f.grid is not None for f in allf) else None
        return (*out, rope)

    def tokenize_multimodal(self, messages: list[dict], images: tp.Sequence[tp.Any] | None = None, **template_kw):
        if self.tokenizer is None:
            raise ValueError("tokenize_multimodal needs a tokenizer with a chat template")
        if images is None:
            images, _ = self.extract_media_from_messages(messages)
        text = self.tokenizer.apply_chat_template(self.normalize_messages(messages), tokenize=False,
                                                  add_generation_prompt=True, **template_kw)
        ids = self.tokenizer(text, add_special_tokens=False)["input_ids"]
        return self.prepare(ids, images)

    def clear_cache(self) -> None:
        if self.cache is not None:
            self.cache.clear()

    def get_cache_stats(self) -> dict | None:
        return None if self.cache is None else self.cache.get_stats()
