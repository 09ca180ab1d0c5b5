"""Multimodal (image → text) models on top of the language models of this package.

``BaseXModalToTextModel`` adds what the reference's base class has (``models/multi_modal/base_model.py:31``):
``update_modal_to_text`` scatters encoder outputs into the text embeddings at the positions the processor recorded.
``ImageToTextModel`` is a complete small architecture in that mould: a ViT encoder (patch projection, pre-norm
transformer blocks), a two-layer projector into the language model's hidden size, and any ``…ForCausalLM`` of this
package as the decoder. Generation splices the image features during prefill through the generator's
``input_embeds_hook``.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...tools.register import MindFormerModuleType, MindFormerRegister
from ..configuration_utils import PretrainedConfig
from ..modeling_utils import PreTrainedModel


class VisionConfig(PretrainedConfig):
    """Vision tower settings: image and patch size, width, depth, heads, MLP width."""

    model_type = "vit"

    @classmethod
    def default_values(cls):
        return dict(image_size=224, patch_size=14, hidden_size=1024, num_hidden_layers=24, num_attention_heads=16,
                    intermediate_size=4096, layer_norm_eps=1e-5, num_channels=3, use_cls_token=True,
                    select_layer=-1)


class ViTBlock(nn.Module):
    """Pre-LN vision transformer block (bidirectional attention + GELU MLP)."""

    def __init__(self, c: VisionConfig, dtype):
        super().__init__()
        h = c.hidden_size
        self.heads = c.num_attention_heads
        self.norm1 = nn.LayerNorm(h, eps=c.layer_norm_eps, dtype=dtype)
        self.qkv = nn.Linear(h, 3 * h, dtype=dtype)
        self.proj = nn.Linear(h, h, dtype=dtype)
        self.norm2 = nn.LayerNorm(h, eps=c.layer_norm_eps, dtype=dtype)
        self.fc1 = nn.Linear(h, c.intermediate_size, dtype=dtype)
        self.fc2 = nn.Linear(c.intermediate_size, h, dtype=dtype)

    def forward(self, x):
        B, N, H = x.shape
        q, k, v = self.qkv(self.norm1(x)).view(B, N, 3, self.heads, H // self.heads).permute(2, 0, 3, 1, 4)
        a = F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(B, N, H)
        x = x + self.proj(a)
        return x + self.fc2(F.gelu(self.fc1(self.norm2(x))))


class ViTEncoder(nn.Module):
    """``pixel_values [N, 3, S, S]`` → patch features ``[N, (S/p)², hidden]`` (the class token is dropped)."""

    def __init__(self, config: VisionConfig, dtype=torch.float32):
        super().__init__()
        c = self.config = config
        self.patch = nn.Conv2d(c.num_channels, c.hidden_size, c.patch_size, c.patch_size, bias=False, dtype=dtype)
        self.num_patches = (c.image_size // c.patch_size) ** 2
        self.cls = nn.Parameter(torch.zeros(1, 1, c.hidden_size, dtype=dtype)) if c.use_cls_token else None
        self.pos = nn.Parameter(torch.randn(1, self.num_patches + int(c.use_cls_token), c.hidden_size, dtype=dtype) * 0.02)
        self.pre_norm = nn.LayerNorm(c.hidden_size, eps=c.layer_norm_eps, dtype=dtype)
        self.blocks = nn.ModuleList([ViTBlock(c, dtype) for _ in range(c.num_hidden_layers)])

    def forward(self, pixel_values):
        x = self.patch(pixel_values.to(self.patch.weight.dtype)).flatten(2).transpose(1, 2)
        if self.cls is not None:
            x = torch.cat([self.cls.expand(x.shape[0], -1, -1), x], dim=1)
        x = self.pre_norm(x + self.pos)
        last = len(self.blocks) + self.config.select_layer + 1 if self.config.select_layer < 0 else self.config.select_layer
        for blk in self.blocks[:last]:
            x = blk(x)
        return x[:, 1:] if self.cls is not None else x


class BaseXModalToTextModel(nn.Module):
    """Mixin-style base: holds ``llm_model`` (a ``PreTrainedModel``) and splices modal features into its embeddings."""

    def __init__(self):
        super().__init__()
        self.llm_model: Optional[PreTrainedModel] = None

    def text_embeddings(self, input_ids: torch.Tensor) -> torch.Tensor:
        emb = self.llm_model.model.embedding.word_embeddings
        if getattr(emb, "tp", 1) > 1:
            raise NotImplementedError("multimodal splicing needs an unsharded embedding table (tensor parallel = 1)")
        return F.embedding(input_ids, emb.weight)

    @staticmethod
    def update_modal_to_text(modal_embeds: torch.Tensor, text_embeds: torch.Tensor,
                             modal_context_pos: torch.Tensor) -> torch.Tensor:
        """``modal_embeds [n, L, H]`` go to ``text_embeds[b, p]`` for every ``(b, p)`` of ``modal_context_pos [n, L,
        2]``."""
        pos = modal_context_pos.reshape(-1, 2).to(text_embeds.device)
        out = text_embeds.clone()
        out[pos[:, 0], pos[:, 1]] = modal_embeds.reshape(-1, modal_embeds.shape[-1]).to(out.dtype)
        return out

    def kvcache(self, layer_idx):
        return self.llm_model.kvcache(layer_idx) if hasattr(self.llm_model, "kvcache") else None


class ImageToTextConfig(PretrainedConfig):
    """Configuration of ``ImageToTextModel``: ``vision_config``, ``text_config`` (any registered causal-LM
    configuration), projector width and the id of the image placeholder token."""

    model_type = "image_to_text"

    @classmethod
    def default_values(cls):
        return dict(vision_config=None, text_config=None, image_pad_token_id=None, projector_hidden_size=None,
                    freeze_vision=False, freeze_llm=False)


@MindFormerRegister.register(MindFormerModuleType.MODELS)
class ImageToTextModel(BaseXModalToTextModel):
    """ViT encoder + MLP projector + causal language model.

    ``forward(input_ids, images, image_context_pos, labels)`` → loss (or logits without labels).
    ``generate(input_ids=…, images=…, image_context_pos=…)`` → token ids, through the language model's generator.
    """
    config_class = ImageToTextConfig

    def __init__(self, config: ImageToTextConfig, llm_model: Optional[PreTrainedModel] = None, device=None, dtype=None):
        super().__init__()
        self.config = config
        vc = config.vision_config if isinstance(config.vision_config, VisionConfig) else VisionConfig(
            **(config.vision_config or {}))
        if llm_model is None:
            from ..auto import AutoModel
            llm_model = AutoModel.from_config(dict(config.text_config), device=device, dtype=dtype)
        self.llm_model = llm_model
        p = next(llm_model.parameters())
        self.vision_encoder = ViTEncoder(vc, dtype=p.dtype).to(p.device)
        lh = llm_model.config.hidden_size
        mid = config.projector_hidden_size or lh
        self.projector = nn.Sequential(nn.Linear(vc.hidden_size, mid, dtype=p.dtype), nn.GELU(),
                                       nn.Linear(mid, lh, dtype=p.dtype)).to(p.device)
        self.num_image_tokens = self.vision_encoder.num_patches
        if config.freeze_vision:
            self.vision_encoder.requires_grad_(False)
        if config.freeze_llm:
            self.llm_model.requires_grad_(False)
        self._pending = None

    def encode_images(self, images: torch.Tensor) -> torch.Tensor:
        p = next(self.projector.parameters())
        return self.projector(self.vision_encoder(images.to(p.device)))

    def forward(self, input_ids, images=None, image_context_pos=None, labels=None, loss_mask=None, **kw):
        embeds = self.text_embeddings(input_ids)
        if images is not None and image_context_pos is not None and image_context_pos.numel():
            embeds = self.update_modal_to_text(self.encode_images(images), embeds, image_context_pos)
        return self.llm_model(input_ids, labels=labels, loss_mask=loss_mask, input_embeds=embeds)

    @torch.no_grad()
    def generate(self, input_ids, images=None, image_context_pos=None, **kwargs):
        """Rows of ``input_ids`` may be lists of different lengths; ``image_context_pos`` indexes (row, position)."""
        llm = self.llm_model
        rows = input_ids.tolist() if torch.is_tensor(input_ids) else [list(r) for r in input_ids]
        feats = None
        if images is not None and image_context_pos is not None and len(image_context_pos):
            feats = self.encode_images(torch.as_tensor(images))
            pos = torch.as_tensor(image_context_pos).reshape(-1, 2)
            starts = [0]
            for r in rows:
                starts.append(starts[-1] + len(r))
            flat_index = torch.tensor([starts[int(b)] + int(p) for b, p in pos.tolist()], dtype=torch.int64)
            feats = feats.reshape(-1, feats.shape[-1])

        def hook(flat, positions, prefill):
            # the generator flattens the prompts in row order for the (single, unchunked) prefill call
            if not prefill or feats is None:
                return None
            emb = self.text_embeddings(flat)
            emb[flat_index.to(emb.device)] = feats.to(emb.dtype)
            return emb.unsqueeze(0)

        llm.input_embeds_hook = hook
        try:
            return llm.generate(rows, **kwargs)
        finally:
            llm.input_embeds_hook = None
