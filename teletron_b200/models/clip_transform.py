"""CLIP feature extractors with the interfaces of ``teletron/models/hunyuanvideo/clip_transform.py``.

* :class:`CLIPTransform` (``:11-87``): text and / or image features of a full CLIP model, either the projected and
  L2-normalised embeddings (``*_w_proj=True``) or the pooled tower outputs.
* :class:`CLIPTextTransform` (``:90-141``): one text tower; ``mode="after_pool"`` gives the pooled vector,
  ``"before_pool"`` the per-token states padded to the model length.
* :class:`CLIPTextWithProjectionTransform` (``:144-227``): two towers (``text_encoder`` + ``text_encoder_2``): penultimate
  hidden states concatenated on the feature dim - the end-of-text token's row for ``"after_pool"``, all tokens for
  ``"before_pool"`` - plus the second tower's projected pooled embedding.

All load lazily.  With ``model_path`` the Hugging Face weights, tokenizer and image processor are used; without it the
models are built from ``config`` with random weights, prompts go through a hashing tokenizer and images through a plain
resize / centre-crop / normalise, which is what the tests use (no weights ship with the package).
"""

from __future__ import annotations

from typing import Optional, Sequence

import torch
import torch.nn.functional as F

from .text_encoders import HashTokenizer, clip_text_config

CLIP_MEAN = (0.48145466, 0.4578275, 0.40821073)
CLIP_STD = (0.26862954, 0.26130258, 0.27577711)


def _dtype(dtype, device):
    if dtype is None:
        return torch.float16 if (device is not None and "cuda" in str(device)) else torch.float32
    return getattr(torch, dtype) if isinstance(dtype, str) else dtype


def _out(t: torch.Tensor, to_numpy: bool):
    return t.contiguous().float().cpu().numpy() if to_numpy else t


def preprocess_images(images: torch.Tensor, size: int = 224) -> torch.Tensor:
    """``[B, 3, H, W]`` RGB in [0, 1] -> resized (short edge ``size``, bicubic), centre-cropped, CLIP-normalised."""
    B, C, H, W = images.shape
    scale = size / min(H, W)
    nh, nw = max(size, round(H * scale)), max(size, round(W * scale))
    x = F.interpolate(images.float(), size=(nh, nw), mode="bicubic", align_corners=False).clamp(0, 1)
    t, l = (nh - size) // 2, (nw - size) // 2
    x = x[:, :, t:t + size, l:l + size]
    mean = torch.tensor(CLIP_MEAN, device=x.device).view(1, 3, 1, 1)
    std = torch.tensor(CLIP_STD, device=x.device).view(1, 3, 1, 1)
    return (x - mean) / std


class _Lazy:
    def __init__(self, model_path: Optional[str], device=None, dtype=None, config=None, max_length: int = 77):
        self.model_path, self.device, self.dtype = model_path, device, _dtype(dtype, device)
        self.config, self.max_length = config, max_length
        self.tokenizer = None
        self._hash = None

    def _place(self, model):
        model.requires_grad_(False)
        return model.to(self.device).to(self.dtype).eval() if self.device is not None else model.to(self.dtype).eval()

    def _tokenize(self, text, pad_to_max: bool, tokenizer=None, hasher=None):
        texts = [text] if isinstance(text, str) else list(text)
        tokenizer = tokenizer or self.tokenizer
        if tokenizer is not None:
            t = tokenizer(text=texts, padding="max_length" if pad_to_max else True, truncation=True, return_tensors="pt")
            return t.input_ids
        ids, mask = (hasher or self._hash)(texts, self.max_length)
        if not pad_to_max:
            ids = ids[:, : int(mask.sum(1).max())]
        return ids


class CLIPTransform(_Lazy):
    def load_model(self):
        if getattr(self, "model", None) is not None:
            return
        from transformers import CLIPModel
        if self.model_path:
            from transformers import CLIPProcessor
            self.processor = CLIPProcessor.from_pretrained(self.model_path)
            self.tokenizer = self.processor.tokenizer
            self.model = self._place(CLIPModel.from_pretrained(self.model_path))
        else:
            self.processor = None
            self.model = self._place(CLIPModel(self.config))
            tc = self.config.text_config
            self.max_length = tc.max_position_embeddings
            # CLIP pools at the position of the largest token id: the stand-in tokenizer ends every prompt with it
            self._hash = HashTokenizer(tc.vocab_size - 1, self.max_length, pad_id=0, eos_id=tc.vocab_size - 1)

    @torch.no_grad()
    def __call__(self, text=None, image=None, text_w_proj: bool = True, image_w_proj: bool = True, to_numpy: bool = True):
        """``image``: ``[B, 3, H, W]`` RGB in [0, 1] (or whatever the Hugging Face processor accepts when weights are loaded)."""
        self.load_model()
        results = []
        if text is not None:
            ids = self._tokenize(text, pad_to_max=False).to(self.model.device)
            if text_w_proj:
                f = self.model.get_text_features(ids)
                f = f.pooler_output if hasattr(f, "pooler_output") else f
                f = f / f.norm(p=2, dim=-1, keepdim=True)
            else:
                f = self.model.text_model(ids)[1]
            results.append(_out(f, to_numpy))
        if image is not None:
            if self.processor is not None:
                px = self.processor(images=image, return_tensors="pt").pixel_values
            else:
                px = preprocess_images(image, self.config.vision_config.image_size)
            px = px.to(self.model.device, self.dtype)
            if image_w_proj:
                f = self.model.get_image_features(px)
                f = f.pooler_output if hasattr(f, "pooler_output") else f
                f = f / f.norm(p=2, dim=-1, keepdim=True)
            else:
                f = self.model.vision_model(px)[1]
            results.append(_out(f, to_numpy))
        if not results:
            return None
        return results if len(results) > 1 else results[0]


class CLIPTextTransform(_Lazy):
    def load_model(self):
        if getattr(self, "text_encoder", None) is not None:
            return
        from transformers import CLIPTextModel
        if self.model_path:
            from transformers import CLIPTokenizer
            self.tokenizer = CLIPTokenizer.from_pretrained(self.model_path)
            self.text_encoder = self._place(CLIPTextModel.from_pretrained(self.model_path))
        else:
            cfg = self.config or clip_text_config(max_len=self.max_length)
            self.max_length = cfg.max_position_embeddings
            self.text_encoder = self._place(CLIPTextModel(cfg))
            self._hash = HashTokenizer(cfg.vocab_size - 1, self.max_length, pad_id=0, eos_id=cfg.vocab_size - 1)

    @torch.no_grad()
    def __call__(self, text, mode: str, to_numpy: bool = True):
        self.load_model()
        if mode not in ("after_pool", "before_pool"):
            raise ValueError(f"mode must be 'after_pool' or 'before_pool', got {mode!r}")
        ids = self._tokenize(text, pad_to_max=mode == "before_pool").to(self.text_encoder.device)
        out = self.text_encoder(ids)
        return _out(out[1] if mode == "after_pool" else out[0], to_numpy)


class CLIPTextWithProjectionTransform(_Lazy):
    """``config``: a pair of text configs (tower one, tower two with projection) when no weights are given."""

    def load_model(self):
        if getattr(self, "text_encoders", None) is not None:
            return
        from transformers import CLIPTextModel, CLIPTextModelWithProjection
        if self.model_path:
            from transformers import CLIPTokenizer
            self.tokenizers = [CLIPTokenizer.from_pretrained(self.model_path, subfolder=s) for s in ("tokenizer", "tokenizer_2")]
            towers = [CLIPTextModel.from_pretrained(self.model_path, subfolder="text_encoder"),
                      CLIPTextModelWithProjection.from_pretrained(self.model_path, subfolder="text_encoder_2")]
            self._hashes = [None, None]
        else:
            c1, c2 = self.config
            self.tokenizers = [None, None]
            towers = [CLIPTextModel(c1), CLIPTextModelWithProjection(c2)]
            self.max_length = c1.max_position_embeddings
            self._hashes = [HashTokenizer(c.vocab_size - 1, c.max_position_embeddings, pad_id=0, eos_id=c.vocab_size - 1) for c in (c1, c2)]
        self.text_encoders = [self._place(t) for t in towers]

    @torch.no_grad()
    def __call__(self, text, mode: str, to_numpy: bool = True):
        self.load_model()
        if mode not in ("after_pool", "before_pool"):
            raise ValueError(f"mode must be 'after_pool' or 'before_pool', got {mode!r}")
        feats, pooled = [], None
        for tok, hasher, enc in zip(self.tokenizers, self._hashes, self.text_encoders):
            ids = self._tokenize(text, pad_to_max=mode == "before_pool", tokenizer=tok, hasher=hasher).to(enc.device)
            out = enc(ids, output_hidden_states=True)
            pooled = out[0]                                  # the pooled output of the final tower is the one returned
            h = out.hidden_states[-2]
            if mode == "after_pool":                         # the end-of-text token (largest id) of every prompt
                h = h[torch.arange(h.shape[0], device=h.device), ids.to(torch.int).argmax(dim=-1)]
            feats.append(h)
        return _out(torch.cat(feats, dim=-1), to_numpy), _out(pooled, to_numpy)
