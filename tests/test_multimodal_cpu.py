"""Multimodal content builders, image processor, ImageToTextModel forward/backward and generation, pipeline."""
import numpy as np
import pytest
import torch

from mindformers_b200.models import AutoModel, ByteTokenizer
from mindformers_b200.models.multi_modal import (BaseImageContentBuilder, BaseImageToTextImageProcessor,
                                                 BaseXModalToTextProcessor, BaseXModalToTextTransform,
                                                 ImageToTextConfig, ImageToTextModel, ModalContentBuilder,
                                                 ModalContentTransformTemplate)
from mindformers_b200.pipeline import pipeline


class ImgTokenizer(ByteTokenizer):
    """Byte tokenizer with three extra ids for the image markers."""
    MARK = {"<img>": 260, "</img>": 261, "<imgpad>": 262}

    def __init__(self, **kw):
        super().__init__(**kw)
        self.vocab_size = 263

    def convert_tokens_to_ids(self, tok):
        return self.MARK.get(tok)

    def decode(self, ids, **kw):
        return super().decode([i for i in ids if i < 260], **kw)

    def encode(self, text, add_special_tokens=True, **kw):
        ids, i = [], 0
        while i < len(text):
            for m, v in self.MARK.items():
                if text.startswith(m, i):
                    ids.append(v)
                    i += len(m)
                    break
            else:
                ids += [b + self.offset for b in text[i].encode()]
                i += 1
        return ([self.bos_token_id] if add_special_tokens and self.add_bos_token else []) + ids


def tiny_model():
    text = dict(model_type="llama", vocab_size=263, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=256, params_dtype="float32")
    vision = dict(image_size=28, patch_size=14, hidden_size=32, num_hidden_layers=2, num_attention_heads=4,
                  intermediate_size=64)
    torch.manual_seed(0)
    return ImageToTextModel(ImageToTextConfig(vision_config=vision, text_config=text, image_pad_token_id=262),
                            device="cpu")


def template(tok, mode="predict", max_length=64):
    proc = BaseImageToTextImageProcessor(image_size=28)
    b = BaseImageContentBuilder("<imgpad>", context_length=4, image_processor=proc, modal_content_max_size=2)
    return ModalContentTransformTemplate(tokenizer=tok, modal_builders={"image": b}, mode=mode, max_length=max_length)


def test_find_tag_and_padding_context():
    assert ModalContentBuilder.find_tag_and_extract("a<img>x.png</img>b<img>y</img>", "<img>", "</img>") == ["x.png", "y"]
    with pytest.raises(ValueError):
        ModalContentBuilder.find_tag_and_extract("<img>x", "<img>", "</img>")
    tok = ImgTokenizer()
    t = template(tok)
    b = t.modal_builders["image"]
    ids = tok.encode("hi<img>p</img>!", add_special_tokens=False)
    padded = b.padding_context(ids, {})
    assert padded.count(262) == 4 and padded[padded.index(260) + 5] == 261
    pos = b.generate_context_positions(padded, batch_index=3)
    assert pos.shape == (1, 4, 2) and (pos[..., 0] == 3).all() and pos[0, :, 1].tolist() == list(range(3, 7))


def test_image_processor_shapes_and_normalisation():
    proc = BaseImageToTextImageProcessor(image_size=28, mean=(0.5, 0.5, 0.5), std=(0.5, 0.5, 0.5))
    img = (np.ones((40, 60, 3)) * 255).astype(np.uint8)
    out = proc(img)
    assert out.shape == (1, 3, 28, 28) and torch.allclose(out, torch.ones_like(out), atol=1e-5)
    from PIL import Image
    out = proc([Image.fromarray(img), torch.zeros(3, 28, 28)])
    assert out.shape == (2, 3, 28, 28) and torch.allclose(out[1], -torch.ones(3, 28, 28))


def test_train_transform_and_model_step():
    tok = ImgTokenizer(add_bos_token=False)
    t = template(tok, mode="train", max_length=48)
    tf = BaseXModalToTextTransform(tok, t)
    img = np.random.default_rng(0).integers(0, 255, (28, 28, 3), dtype=np.uint8)
    b = t.modal_builders["image"]
    b.load_image = lambda item: img                     # tags name files; the test supplies the pixels directly
    rec = tf([{"from": "user", "value": "<img>a.png</img>what?"}, {"from": "assistant", "value": "cat"}])
    assert len(rec["input_ids"]) == len(rec["labels"]) == 47
    kept = [l for l in rec["labels"] if l != -100]
    assert kept == tok.encode("cat", add_special_tokens=False) + [tok.eos_token_id]
    assert rec["image_context_pos"].shape == (2, 4, 2)         # padded to modal_content_max_size in train mode
    batch = t.batch([rec, rec])
    model = tiny_model()
    # one image per sample here: use the first position block of each record
    pos = torch.stack([torch.from_numpy(rec["image_context_pos"][0]) for _ in range(2)])
    pos[1, :, 0] = 1
    loss = model(batch["input_ids"], images=batch["images"], image_context_pos=pos, labels=batch["labels"])
    loss.backward()
    assert torch.isfinite(loss)
    assert model.projector[0].weight.grad.abs().sum() > 0 and model.vision_encoder.patch.weight.grad.abs().sum() > 0
    # the image changes the loss
    loss2 = model(batch["input_ids"], images=batch["images"] * 0, image_context_pos=pos, labels=batch["labels"])
    assert abs(loss.item() - loss2.item()) > 1e-6


def test_generate_matches_forward_and_pipeline():
    tok = ImgTokenizer()
    model = tiny_model().eval()
    proc = BaseXModalToTextProcessor(template(tok), tokenizer=tok)
    img = np.random.default_rng(1).integers(0, 255, (28, 28, 3), dtype=np.uint8)
    query = [{"image": img}, {"text": "describe"}]
    batch = proc(query)
    assert batch["images"].shape == (1, 3, 28, 28) and batch["image_context_pos"].shape == (1, 4, 2)
    out = model.generate(batch["input_ids_list"], images=batch["images"], image_context_pos=batch["image_context_pos"],
                         max_new_tokens=3, do_sample=False)
    prompt = batch["input_ids_list"][0]
    assert out[0][:len(prompt)] == prompt and len(out[0]) <= len(prompt) + 3
    with torch.no_grad():
        logits = model(torch.tensor([prompt]), images=batch["images"], image_context_pos=batch["image_context_pos"])
    assert out[0][len(prompt)] == int(logits[-1, :263].argmax())
    no_img = model.generate([prompt], max_new_tokens=1, do_sample=False)
    with torch.no_grad():
        plain = model.llm_model(torch.tensor([prompt]))
    assert no_img[0][len(prompt)] == int(plain[-1, :263].argmax())
    pipe = pipeline("multi_modal_to_text_generation", model=model, processor=proc, max_new_tokens=3, do_sample=False)
    res = pipe([query])
    assert isinstance(res[0]["text_generation_text"][0], str)
