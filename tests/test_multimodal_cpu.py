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


def test_modal_to_text_sft_dataset_llava_handler_and_s3_paths(tmp_path):
    import json
    from mindformers_b200.dataset import LlavaInstructDataHandler, ModalToTextSFTDataset
    from mindformers_b200.dataset import utils_s3
    tok = ImgTokenizer(add_bos_token=False)
    t = template(tok, mode="train", max_length=48)
    img = np.random.default_rng(0).integers(0, 255, (28, 28, 3), dtype=np.uint8)
    seen = []
    t.modal_builders["image"].load_image = lambda item: (seen.append(item), img)[1]
    records = [{"conversations": [["user", "<img>a.png</img>what?"], ["assistant", "cat"]]},
               {"image": "b.png", "conversations": [{"from": "human", "value": "<image>\\nand this?"},
                                                    {"from": "gpt", "value": "dog"}]}]
    ann = tmp_path / "ann.json"
    json.dump(records, open(ann, "w"))
    loader = ModalToTextSFTDataset(dict(annotation_file=str(ann), modal_content_transform_template=t, batch_size=2,
                                        image_dir=str(tmp_path / "imgs")))
    batch = next(iter(loader))
    assert batch["input_ids"].shape == (2, 47) and batch["labels"].shape == (2, 47)
    assert seen[0] == "a.png" and seen[1] == str(tmp_path / "imgs" / "b.png")
    pos = batch["image_context_pos"]
    assert pos.shape[-1] == 2 and set(pos[..., 0].unique().tolist()) == {0, 1}         # rows of the batch
    kept = [l for l in batch["labels"][1].tolist() if l != -100]
    assert kept == tok.encode("dog", add_special_tokens=False) + [tok.eos_token_id]

    h = LlavaInstructDataHandler(tok, seq_length=80, image_dir="/data/img", image_token_num=3)
    out = h.handle_one(records[1])
    assert out["image_path"] == "/data/img/b.png" and out["input_ids"].shape == (81,)
    text = tok.decode([i for i in out["input_ids"].tolist() if i != (tok.pad_token_id or 0)])
    assert text.count("<image>") == 3 and "ASSISTANT: dog" in text
    assert [l for l in out["labels"].tolist() if l != -100][-1] == tok.eos_token_id

    assert utils_s3.is_s3_path("s3://bucket/a/b.idx") and not utils_s3.is_s3_path("/data/b.idx")
    assert utils_s3.parse_s3_path("s3://bucket/a/b.idx") == ("bucket", "a/b.idx")

    class FakeS3:
        store = {("bucket", "a/b.idx"): b"0123456789"}
        downloads = 0

        def head_object(self, Bucket, Key):
            return {"ContentLength": len(self.store[(Bucket, Key)])}

        def download_file(self, bucket, key, dst):
            FakeS3.downloads += 1
            open(dst, "wb").write(self.store[(bucket, key)])

        def get_object(self, Bucket, Key, Range):
            a, b = (int(x) for x in Range.split("=")[1].split("-"))
            return {"Body": self.store[(Bucket, Key)][a:b + 1]}

    cfg = utils_s3.S3Config(path_to_idx_cache=str(tmp_path / "cache"))
    local = utils_s3.maybe_download_index("s3://bucket/a/b.idx", cfg, FakeS3())
    assert open(local, "rb").read() == b"0123456789"
    utils_s3.maybe_download_index("s3://bucket/a/b.idx", cfg, FakeS3())
    assert FakeS3.downloads == 1                                                       # second call hits the cache
    assert utils_s3.object_exists("s3://bucket/a/b.idx", FakeS3()) and not utils_s3.object_exists("s3://bucket/x", FakeS3())
    assert utils_s3.read_range("s3://bucket/a/b.idx", 2, 4, FakeS3()) == b"2345"
    assert utils_s3.maybe_download_index("/local/file.idx", cfg) == "/local/file.idx"


def test_multimodal_trainer_predict_from_records(tmp_path):
    """The task trainer turns conversation records into tensors with the processor, generates and writes the texts."""
    from mindformers_b200.tools.register import MindFormerConfig
    from mindformers_b200.trainer.base_trainer import MultiModalToTextGenerationTrainer
    tok = ImgTokenizer()
    model = tiny_model().eval()
    proc = BaseXModalToTextProcessor(template(tok), tokenizer=tok)
    img = np.random.default_rng(2).integers(0, 255, (28, 28, 3), dtype=np.uint8)
    cfg = MindFormerConfig({"run_mode": "predict", "save_file": str(tmp_path / "out.txt")})
    trainer = MultiModalToTextGenerationTrainer(model_name="tiny")
    res = trainer.predict(cfg, input_data=[[{"image": img}, {"text": "what is this"}]], network=model, tokenizer=tok,
                          processor=proc, max_new_tokens=3, do_sample=False)
    assert isinstance(res[0]["text_generation_text"][0], str)
    assert (tmp_path / "out.txt").read_text().strip()
    one = trainer.predict(cfg, input_data=[{"image": img}, {"text": "and this"}], network=model, tokenizer=tok,
                          processor=proc, max_new_tokens=2, do_sample=False)
    assert len(one) == 1


def test_features_travel_through_shared_memory_as_two_negative_ids(tmp_path):
    """The serving front end parks an array in shared memory and sends (encoded name, encoded shape); the worker gets
    the same array back; corrupted or ordinary negative values are rejected; the clean-up file unlinks leftovers."""
    import numpy as np
    import pytest
    from mindformers_b200.models.multi_modal.shm_utils import (SHM_NAME_PREFIX, decode_shape_from_int64,
                                                               decode_shm_name_from_int64, encode_shape_to_int64,
                                                               encode_shm_name_to_int64, get_data_from_shm, put_data_to_shm,
                                                               release_shared_memory)
    from mindformers_b200.models.multi_modal.utils import DataRecord
    for shape in ((7,), (2, 3), (4, 3, 336, 336), (2, 5, 3, 224, 224), (1, 2, 3, 4, 5, 6)):
        code = encode_shape_to_int64(shape)
        assert code < 0 and -code < 2 ** 63 and decode_shape_from_int64(code) == shape
    for name in (SHM_NAME_PREFIX + "1a2b3c4d", SHM_NAME_PREFIX + "00ff00ff00", SHM_NAME_PREFIX + "7"):
        code = encode_shm_name_to_int64(name)
        assert code < 0 and -code < 2 ** 63 and decode_shm_name_from_int64(code) == name
    with pytest.raises(ValueError):
        decode_shape_from_int64(encode_shape_to_int64((2, 3)) - 1)
    with pytest.raises(ValueError):
        decode_shm_name_from_int64(-123456)
    with pytest.raises(ValueError):
        encode_shape_to_int64((1 << 30, 1 << 30, 3))
    feats = np.random.default_rng(0).standard_normal((2, 3, 8, 8)).astype(np.float32)
    book = str(tmp_path / "segments.txt")
    name_id, shape_id = put_data_to_shm(feats, book)
    assert name_id < 0 and shape_id < 0
    np.testing.assert_array_equal(get_data_from_shm(name_id, shape_id, np.float32), feats)
    put_data_to_shm(feats, book)                        # a segment nobody fetches
    assert release_shared_memory(book) == 1             # the first one is gone already, the second is unlinked here
    rec = DataRecord()
    rec.put("ids", 1, append=True)
    rec.put("ids", 2, append=True)
    rec.put_from_dict({"n": 3})
    assert rec.output(["ids", "n"], "tuple") == ([1, 2], 3) and rec.has_key("n") and rec.output(["n"]) == {"n": 3}
