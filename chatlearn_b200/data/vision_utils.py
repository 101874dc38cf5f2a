"""Image preprocessing for vision-language prompts.

Parity: chatlearn/data/vision_utils.py and the processor calls in
chatlearn/data/vl_prompt_dataset.py (the reference delegates to the HuggingFace Qwen2-VL image
processor and ``qwen_vl_utils``).  Implemented here from the published recipe:

* ``smart_resize``: both sides become multiples of ``patch · merge`` (28), the aspect ratio is kept
  as far as the pixel budget ``[min_pixels, max_pixels]`` allows;
* bicubic resize, scale to [0, 1], normalise with the CLIP mean / std;
* a still image is repeated ``temporal_patch_size`` times; patches of ``C × Tp × P × P`` values are
  emitted merge-block by merge-block (the order the vision tower's window logic expects);
* ``image_grid_thw = (1, H / P, W / P)``; the prompt holds ``grid_t · grid_h · grid_w / merge²`` image
  placeholder tokens per image.
"""
import io
import math
from typing import List, Optional, Sequence, Tuple

import torch

CLIP_MEAN = (0.48145466, 0.4578275, 0.40821073)
CLIP_STD = (0.26862954, 0.26130258, 0.27577711)


def smart_resize(height: int, width: int, factor: int = 28, min_pixels: int = 56 * 56,
                 max_pixels: int = 14 * 14 * 4 * 1280) -> Tuple[int, int]:
    if max(height, width) / min(height, width) > 200:
        raise ValueError("aspect ratio above 200 is not supported")
    h = max(factor, round(height / factor) * factor)
    w = max(factor, round(width / factor) * factor)
    if h * w > max_pixels:
        beta = math.sqrt(height * width / max_pixels)
        h = max(factor, math.floor(height / beta / factor) * factor)
        w = max(factor, math.floor(width / beta / factor) * factor)
    elif h * w < min_pixels:
        beta = math.sqrt(min_pixels / (height * width))
        h = math.ceil(height * beta / factor) * factor
        w = math.ceil(width * beta / factor) * factor
    return h, w


def load_image(src):
    """PIL image from a path, raw bytes, a hex string of bytes, a dict with ``path``/``bytes``, an ``[H, W, 3]``
    uint8 array (a decoded video frame), or a PIL image."""
    from PIL import Image
    if isinstance(src, Image.Image):
        return src.convert("RGB")
    if hasattr(src, "shape") and hasattr(src, "dtype") and len(src.shape) == 3:
        import numpy as np
        return Image.fromarray(np.asarray(src, dtype=np.uint8)).convert("RGB")
    if isinstance(src, dict):
        src = src.get("bytes") or src.get("path")
    if isinstance(src, str):
        try:
            raw = bytes.fromhex(src)
            return Image.open(io.BytesIO(raw)).convert("RGB")
        except ValueError:
            return Image.open(src).convert("RGB")
    if isinstance(src, (bytes, bytearray)):
        return Image.open(io.BytesIO(src)).convert("RGB")
    raise TypeError(f"cannot load an image from {type(src).__name__}")


def image_to_patches(img, patch_size: int = 14, temporal_patch_size: int = 2, merge_size: int = 2,
                     min_pixels: int = 56 * 56, max_pixels: int = 14 * 14 * 4 * 1280,
                     mean: Sequence[float] = CLIP_MEAN, std: Sequence[float] = CLIP_STD):
    """Returns ``(pixel_values [grid_h·grid_w, C·Tp·P·P] fp32, (1, grid_h, grid_w))``."""
    import numpy as np
    from PIL import Image
    img = load_image(img)
    W, H = img.size
    h, w = smart_resize(H, W, patch_size * merge_size, min_pixels, max_pixels)
    img = img.resize((w, h), resample=Image.BICUBIC)
    x = torch.from_numpy(np.asarray(img, dtype=np.float32) / 255.0).permute(2, 0, 1)        # [C, h, w]
    x = (x - torch.tensor(mean).view(3, 1, 1)) / torch.tensor(std).view(3, 1, 1)
    frames = x.unsqueeze(0).repeat(temporal_patch_size, 1, 1, 1)                              # [Tp, C, h, w]
    gh, gw, m, P, C = h // patch_size, w // patch_size, merge_size, patch_size, 3
    t = frames.view(1, temporal_patch_size, C, gh // m, m, P, gw // m, m, P)
    t = t.permute(0, 3, 6, 4, 7, 2, 1, 5, 8)        # grid_t, gh/m, gw/m, m, m, C, Tp, P, P
    return t.reshape(gh * gw, C * temporal_patch_size * P * P).contiguous(), (1, gh, gw)


def load_video(path: str, fps: float = 2.0, max_frames: int = 768):
    """Frames of a video file sampled at ``fps`` frames per second (at most ``max_frames``, then evenly thinned) as
    ``([H, W, 3] uint8 arrays, the sampling rate that was reached)``.  Decoding uses OpenCV."""
    try:
        import cv2
    except ImportError as e:                                        # pragma: no cover
        raise RuntimeError("reading video files needs OpenCV (cv2); pass decoded frames instead") from e
    cap = cv2.VideoCapture(path)
    if not cap.isOpened():
        raise FileNotFoundError(f"cannot open video '{path}'")
    native = cap.get(cv2.CAP_PROP_FPS) or 0.0
    step = max(native / fps, 1.0) if native > 0 else 1.0
    frames, want, i = [], 0.0, 0
    while True:
        ok, img = cap.read()
        if not ok:
            break
        if i >= want - 1e-6:
            frames.append(cv2.cvtColor(img, cv2.COLOR_BGR2RGB))
            want += step
        i += 1
    cap.release()
    if not frames:
        raise ValueError(f"video '{path}' holds no frames")
    rate = (native / step) if native > 0 else fps
    if len(frames) > max_frames:
        keep = [int(round(j * (len(frames) - 1) / (max_frames - 1))) for j in range(max_frames)]
        rate *= max_frames / len(frames)
        frames = [frames[j] for j in keep]
    return frames, rate


def video_to_patches(frames, fps: float = 2.0, patch_size: int = 14, temporal_patch_size: int = 2, merge_size: int = 2,
                     min_pixels: int = 56 * 56, max_pixels: int = 14 * 14 * 4 * 320,
                     mean: Sequence[float] = CLIP_MEAN, std: Sequence[float] = CLIP_STD):
    """Frames of one video (paths, bytes, arrays or PIL images, sampled at ``fps`` frames per second) as
    ``(pixel_values [grid_t·grid_h·grid_w, C·Tp·P·P] fp32, (grid_t, grid_h, grid_w), seconds per temporal grid step)``:
    every frame is resized to the size the first one gets, ``Tp`` consecutive frames form one temporal grid step (the
    last frame is repeated to fill the last step), and the patches are ordered like those of an image."""
    import numpy as np
    from PIL import Image
    imgs = [load_image(f) for f in frames]
    assert imgs, "a video needs at least one frame"
    W, H = imgs[0].size
    h, w = smart_resize(H, W, patch_size * merge_size, min_pixels, max_pixels)
    mean_t, std_t = torch.tensor(mean).view(3, 1, 1), torch.tensor(std).view(3, 1, 1)
    xs = []
    for im in imgs:
        x = torch.from_numpy(np.asarray(im.resize((w, h), resample=Image.BICUBIC), dtype=np.float32) / 255.0).permute(2, 0, 1)
        xs.append((x - mean_t) / std_t)
    while len(xs) % temporal_patch_size:
        xs.append(xs[-1])
    x = torch.stack(xs)                                                                      # [T, C, h, w]
    gt, gh, gw, m, P, C = len(xs) // temporal_patch_size, h // patch_size, w // patch_size, merge_size, patch_size, 3
    t = x.view(gt, temporal_patch_size, C, gh // m, m, P, gw // m, m, P)
    t = t.permute(0, 3, 6, 4, 7, 2, 1, 5, 8)        # grid_t, gh/m, gw/m, m, m, C, Tp, P, P
    return t.reshape(gt * gh * gw, C * temporal_patch_size * P * P).contiguous(), (gt, gh, gw), temporal_patch_size / float(fps)


def expand_image_tokens(input_ids: List[int], grids: Sequence[Sequence[int]], image_token_id: int,
                        merge_size: int = 2, video_token_id: Optional[int] = None) -> List[int]:
    """Replace the i-th single image (or video) placeholder by as many placeholders as the i-th item of ``grids``
    (images and videos in the order of their placeholders) has merged patches."""
    out, gi = [], 0
    for tok in input_ids:
        if tok == image_token_id or (video_token_id is not None and tok == video_token_id):
            t, h, w = grids[gi]
            gi += 1
            out.extend([tok] * (t * h * w // (merge_size ** 2)))
        else:
            out.append(tok)
    assert gi == len(grids), f"{len(grids)} images / videos but {gi} placeholders in the prompt"
    return out


def process_visuals(input_ids: List[int], images, videos, image_token_id: int, video_token_id: Optional[int],
                    tokens_per_second: float = 1.0, video_kw=None, **kw):
    """Patches of a prompt's images and videos in the order of their (single) placeholders:
    ``(pixel_values, grids [[t, h, w], ...], time steps per item)``.  ``videos[i]`` is a list of frames,
    ``{"frames": [...], "fps": f}``, a file path or ``{"path": ..., "fps": sampling rate}``; a video's time step is its seconds per temporal grid step x
    ``tokens_per_second`` (``None`` for images)."""
    images, videos = list(images or []), list(videos or [])
    pv, grids, steps, ii, vi = [], [], [], 0, 0
    for tok in input_ids:
        if tok == image_token_id and ii < len(images):
            p, g = image_to_patches(images[ii], **kw)
            ii += 1
            steps.append(None)
        elif video_token_id is not None and tok == video_token_id and vi < len(videos):
            v = videos[vi]
            vi += 1
            if isinstance(v, str) or (isinstance(v, dict) and "path" in v):
                # a video file: decoded and sampled here
                path, target = (v, 2.0) if isinstance(v, str) else (v["path"], float(v.get("fps", 2.0)))
                frames, fps = load_video(path, target, int(v.get("max_frames", 768)) if isinstance(v, dict) else 768)
            else:
                frames, fps = (v["frames"], float(v.get("fps", 2.0))) if isinstance(v, dict) else (v, 2.0)
            p, g, sec = video_to_patches(frames, fps=fps, **{**kw, **(video_kw or {})})
            steps.append(sec * tokens_per_second)
        else:
            continue
        pv.append(p)
        grids.append(list(g))
    assert ii == len(images) and vi == len(videos), \
        f"{len(images)} images and {len(videos)} videos but {ii} and {vi} placeholders in the prompt"
    if not pv:
        return torch.zeros(0, 0), [], []
    return torch.cat(pv, 0), grids, steps


def process_images(images, **kw):
    """``(pixel_values [sum patches, D], image_grid_thw [n, 3])`` of a list of images."""
    pv, grids = [], []
    for im in images:
        p, g = image_to_patches(im, **kw)
        pv.append(p)
        grids.append(g)
    if not pv:
        return torch.zeros(0, 0), torch.zeros(0, 3, dtype=torch.long)
    return torch.cat(pv, 0), torch.tensor(grids, dtype=torch.long)
