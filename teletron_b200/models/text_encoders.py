"""Text encoders for the encoder service: a LLaMA-style decoder for token embeddings and a CLIP text model for the
pooled vector, plus the prompt utilities of the reference.

Covers ``teletron/models/hunyuanvideo/text_encoder.py`` (``PromptEncoder`` with modes ``clip_text`` /
``clip_text_proj`` / ``clip_text_and_proj`` / ``t5`` / ``llama``, ``truncate_prompt``, ``pad_prompt``) and
``clip_transform.py`` (``CLIPTextTransform`` pooled / unpooled).  Models come from the installed ``transformers``
package.  With a ``model_path`` they load pretrained weights and the matching tokenizer; without one (benchmarks,
tests: no network, no checkpoint files) they are built from the architecture config with random weights and fed by
:class:`HashTokenizer`, a deterministic stand-in that maps whitespace-separated words to ids.
"""

from __future__ import annotations

import hashlib
from typing import List, Optional, Sequence, Tuple

import torch


class HashTokenizer:
    """Deterministic word -> id tokenizer with BOS / padding, used when no tokenizer files are available."""

    def __init__(self, vocab_size: int, max_length: int, bos_id: int = 1, pad_id: int = 0, eos_id: Optional[int] = None):
        self.vocab_size, self.max_length, self.bos_id, self.pad_id = vocab_size, max_length, bos_id, pad_id
        self.eos_id = eos_id            # appended to every prompt when set (CLIP pools at its end-of-text token)

    def __call__(self, prompts: Sequence[str], max_length: Optional[int] = None):
        L = max_length or self.max_length
        ids = torch.full((len(prompts), L), self.pad_id, dtype=torch.long)
        mask = torch.zeros(len(prompts), L, dtype=torch.long)
        for i, p in enumerate(prompts):
            toks = [self.bos_id] + [2 + int.from_bytes(hashlib.md5(w.encode()).digest()[:4], "little") % (self.vocab_size - 2)
                                    for w in p.split()]
            toks = toks[:L] if self.eos_id is None else toks[:L - 1] + [self.eos_id]
            ids[i, :len(toks)] = torch.tensor(toks)
            mask[i, :len(toks)] = 1
        return ids, mask


def llama_config(num_layers: int = 32, hidden: int = 4096, heads: int = 32, kv_heads: int = 8, ffn: int = 14336,
                 vocab: int = 128256):
    from transformers import LlamaConfig
    return LlamaConfig(vocab_size=vocab, hidden_size=hidden, intermediate_size=ffn, num_hidden_layers=num_layers,
                       num_attention_heads=heads, num_key_value_heads=kv_heads, max_position_embeddings=8192,
                       rms_norm_eps=1e-5, rope_theta=500000.0)


def clip_text_config(num_layers: int = 12, hidden: int = 768, heads: int = 12, vocab: int = 49408, max_len: int = 77):
    from transformers import CLIPTextConfig
    return CLIPTextConfig(vocab_size=vocab, hidden_size=hidden, intermediate_size=4 * hidden, num_hidden_layers=num_layers,
                          num_attention_heads=heads, max_position_embeddings=max_len, projection_dim=hidden)


class LlamaTextEncoder:
    """``prompts -> (last_hidden_state [B, L, hidden], mask [B, L])`` (mode ``llama`` of the reference's PromptEncoder)."""

    def __init__(self, model_path: Optional[str] = None, max_length: int = 256, device=None, dtype=torch.bfloat16, config=None):
        from transformers import LlamaModel
        self.max_length = max_length
        self.device = device
        if model_path:
            from transformers import AutoTokenizer
            self.model = LlamaModel.from_pretrained(model_path, torch_dtype=dtype).to(device).eval()
            self.tokenizer = AutoTokenizer.from_pretrained(model_path)
            self._hash = None
        else:
            cfg = config or llama_config()
            with torch.device(device or "cpu"):
                self.model = LlamaModel(cfg).to(dtype).eval()
            self.tokenizer = None
            self._hash = HashTokenizer(cfg.vocab_size, max_length)
        for p in self.model.parameters():
            p.requires_grad_(False)

    def tokenize(self, prompts: Sequence[str]):
        if self._hash is not None:
            return self._hash(prompts, self.max_length)
        t = self.tokenizer(list(prompts), padding="max_length", max_length=self.max_length, truncation=True, return_tensors="pt")
        return t.input_ids, t.attention_mask

    @torch.no_grad()
    def __call__(self, prompts: Sequence[str]) -> Tuple[torch.Tensor, torch.Tensor]:
        ids, mask = self.tokenize(prompts)
        ids, mask = ids.to(self.device), mask.to(self.device)
        out = self.model(input_ids=ids, attention_mask=mask)
        return out.last_hidden_state, mask.bool()


class ClipTextEncoder:
    """``prompts -> pooled [B, hidden]`` (``CLIPTextTransform`` with ``pooled=True`` in the reference)."""

    def __init__(self, model_path: Optional[str] = None, max_length: int = 77, device=None, dtype=torch.bfloat16, config=None):
        from transformers import CLIPTextModel
        self.max_length, self.device = max_length, device
        if model_path:
            from transformers import AutoTokenizer
            self.model = CLIPTextModel.from_pretrained(model_path, torch_dtype=dtype).to(device).eval()
            self.tokenizer = AutoTokenizer.from_pretrained(model_path)
            self._hash = None
        else:
            cfg = config or clip_text_config(max_len=max_length)
            with torch.device(device or "cpu"):
                self.model = CLIPTextModel(cfg).to(dtype).eval()
            self.tokenizer = None
            self._hash = HashTokenizer(cfg.vocab_size, max_length, bos_id=cfg.vocab_size - 2, pad_id=cfg.vocab_size - 1)
        for p in self.model.parameters():
            p.requires_grad_(False)

    @torch.no_grad()
    def __call__(self, prompts: Sequence[str], pooled: bool = True) -> torch.Tensor:
        if self._hash is not None:
            ids, mask = self._hash(prompts, self.max_length)
        else:
            t = self.tokenizer(list(prompts), padding="max_length", max_length=self.max_length, truncation=True, return_tensors="pt")
            ids, mask = t.input_ids, t.attention_mask
        out = self.model(input_ids=ids.to(self.device), attention_mask=mask.to(self.device))
        return out.pooler_output if pooled else out.last_hidden_state


def t5_config(num_layers: int = 24, hidden: int = 4096, heads: int = 64, ffn: int = 10240, vocab: int = 32128):
    from transformers import T5Config
    return T5Config(vocab_size=vocab, d_model=hidden, d_kv=hidden // heads, d_ff=ffn, num_layers=num_layers, num_heads=heads,
                    feed_forward_proj="gated-gelu", is_encoder_decoder=False, use_cache=False)


class _HFTextModel:
    """One Hugging Face text model + tokenizer (a hashing stand-in when no weights are given)."""

    def __init__(self, kind: str, model_path: Optional[str], max_length: int, device, dtype, config=None):
        import transformers
        cls = {"clip": transformers.CLIPTextModel, "clip_proj": transformers.CLIPTextModelWithProjection,
               "t5": transformers.T5EncoderModel}[kind]
        self.max_length, self.device = max_length, device
        if model_path:
            self.model = cls.from_pretrained(model_path, torch_dtype=dtype).to(device).eval()
            self.tokenizer = transformers.AutoTokenizer.from_pretrained(model_path)
            self._hash = None
        else:
            cfg = config or (t5_config() if kind == "t5" else clip_text_config(max_len=max_length))
            with torch.device(device or "cpu"):
                self.model = cls(cfg).to(dtype).eval()
            self.tokenizer = None
            self._hash = HashTokenizer(cfg.vocab_size, max_length, pad_id=0)
        for p in self.model.parameters():
            p.requires_grad_(False)

    def tokenize(self, prompts, max_length=None):
        n = max_length or self.max_length
        if self._hash is not None:
            return self._hash(prompts, n)
        t = self.tokenizer(list(prompts), padding="max_length", max_length=n, truncation=True, return_tensors="pt")
        return t.input_ids, t.attention_mask

    def __call__(self, ids, mask, **kw):
        return self.model(input_ids=ids.to(self.device), attention_mask=None if mask is None else mask.to(self.device), **kw)


class PromptEncoder:
    """Lazy-loading front end with the reference's five modes (``text_encoder.py:14-50, 125-238``):

    * ``llama``: last hidden state ``[B, L, hidden]``;
    * ``clip_text``: CLIP text last hidden state ``[B, L, hidden]``;  ``t5``: T5 encoder last hidden state;
    * ``clip_text_proj``: projected pooled CLIP embedding as ``[B, 1, proj]``;
    * ``clip_text_and_proj``: two CLIP towers (``text_encoder`` and ``text_encoder_2`` under ``model_path``): the
      penultimate hidden states concatenated on the feature dim, plus the second tower's projected pooled embedding,
      returned as ``(embeds, pooled)``.

    Returns ``(embeds, masks)``; ``masks`` is ``None`` unless ``with_attention_mask`` (then the masks are also passed to
    the encoders, as in the reference).  Without ``model_path`` the models are built from configs with random weights and a
    hashing tokenizer (``configs``: one config per tower)."""

    MODES = ("llama", "clip_text", "clip_text_proj", "clip_text_and_proj", "t5")

    def __init__(self, mode: str, model_path: Optional[str] = None, device=None, dtype=None, max_length: Optional[int] = None,
                 configs: Optional[Sequence] = None):
        if dtype is None:
            dtype = torch.float16 if (device is not None and "cuda" in str(device)) else torch.float32
        if isinstance(dtype, str):
            dtype = getattr(torch, dtype)
        if mode not in self.MODES:
            raise ValueError(f"Unsupported mode: {mode}")
        self.mode, self.model_path, self.device, self.dtype = mode, model_path, device, dtype
        self.max_length = max_length or (256 if mode in ("llama", "t5") else 77)
        self.configs = list(configs) if configs else None
        self.encoders = None

    def _paths(self):
        import os
        if not self.model_path:
            return [None, None]
        found = [os.path.join(self.model_path, n) for n in ("text_encoder", "text_encoder_2")
                 if os.path.exists(os.path.join(self.model_path, n))]
        return (found or [self.model_path]) + [None]

    def load_model(self):
        if self.encoders is not None:
            return
        paths, cfg = self._paths(), (self.configs or [None, None]) + [None]
        if self.mode == "llama":
            self.encoders = [LlamaTextEncoder(paths[0], self.max_length, self.device, self.dtype, config=cfg[0])]
        elif self.mode == "clip_text_and_proj":
            self.encoders = [_HFTextModel("clip", paths[0], self.max_length, self.device, self.dtype, cfg[0]),
                             _HFTextModel("clip_proj", paths[1], self.max_length, self.device, self.dtype, cfg[1])]
        else:
            kind = {"clip_text": "clip", "clip_text_proj": "clip_proj", "t5": "t5"}[self.mode]
            self.encoders = [_HFTextModel(kind, paths[0], self.max_length, self.device, self.dtype, cfg[0])]

    @torch.no_grad()
    def __call__(self, prompt, max_length: Optional[int] = None, with_attention_mask: bool = False):
        self.load_model()
        prompts = [prompt] if isinstance(prompt, str) else list(prompt)
        if self.mode == "llama":
            enc = self.encoders[0]
            if max_length:
                enc.max_length = max_length
            emb, mask = enc(prompts)
            return emb, (mask if with_attention_mask else None)
        toks = [e.tokenize(prompts, max_length) for e in self.encoders]
        masks = [m for _, m in toks]
        use = (lambda i: masks[i]) if with_attention_mask else (lambda i: None)
        if self.mode == "clip_text_and_proj":
            hidden, pooled = [], None
            for i, e in enumerate(self.encoders):
                out = e(toks[i][0], use(i), output_hidden_states=True)
                pooled = out[0]                         # of interest: the pooled output of the final tower only
                hidden.append(out.hidden_states[-2])
            emb = (torch.cat(hidden, dim=-1), pooled)
        else:
            out = self.encoders[0](toks[0][0], use(0))
            emb = out[0].unsqueeze(1) if self.mode == "clip_text_proj" else out[0]
        if not with_attention_mask:
            return emb, None
        return emb, (masks[0] if len(masks) == 1 else masks)


def truncate_prompt(prompt_embeds, prompt_masks):
    """Drop padded positions (``text_encoder.py:241-248``)."""
    out = [e[: int(m.sum().item())] for e, m in zip(prompt_embeds, prompt_masks)]
    return out[0] if len(out) == 1 else out


def pad_prompt(prompt_embeds: torch.Tensor, max_length: int, prompt_masks: Optional[torch.Tensor] = None):
    """Zero-pad ``[L, C]`` embeddings (and their mask) to ``max_length`` (``text_encoder.py:251-270``)."""
    cur = prompt_embeds.shape[0]
    if cur > max_length:
        raise ValueError(f"prompt of {cur} tokens exceeds max_length {max_length}")
    if prompt_masks is None:
        prompt_masks = torch.ones(cur, device=prompt_embeds.device, dtype=torch.int64)
    if cur == max_length:
        return prompt_embeds, prompt_masks
    e = torch.zeros((max_length,) + tuple(prompt_embeds.shape[1:]), device=prompt_embeds.device, dtype=prompt_embeds.dtype)
    m = torch.zeros(max_length, device=prompt_masks.device, dtype=prompt_masks.dtype)
    e[:cur], m[:cur] = prompt_embeds, prompt_masks
    return e, m
