import pytest
import torch

from hibana_b200.engine import media
from hibana_b200.models.vision import VisionConfig, VisionEncoder

CFG = VisionConfig(image=64, patch=16, width=160, depth=2, heads=2, mlp=320, shuffle=2, out_hidden=256)


def test_encoder_shapes_and_pixel_shuffle_cpu():
    enc = VisionEncoder(CFG, "cpu")
    px = torch.randn(2, 3, 64, 64)
    out = enc.encode(px)
    assert out.shape == (2 * CFG.tokens_per_image, 256) and CFG.tokens_per_image == 4
    # pixel shuffle groups the 2 x 2 neighbours of a cell
    x = torch.arange(16).float().view(16, 1).repeat(1, 160)
    sh = enc.pixel_shuffle(x, 1)
    assert sh.shape == (4, 640) and sh[0, ::160].tolist() == [0, 1, 4, 5] and sh[3, ::160].tolist() == [10, 11, 14, 15]
    # patch order is row-major
    img = torch.zeros(1, 3, 64, 64)
    img[0, :, 16:32, 48:64] = 1.0
    rows = enc.patchify(img)
    assert int(rows.float().sum(1).nonzero()[0]) == 1 * 4 + 3


def test_placeholders_and_splice():
    a, b = media.Image(b"cat", None), media.Image(b"dog", None)
    pa = media.placeholder_ids(a, 4)
    assert all(i < 0 for i in pa) and len(set(pa)) == 4 and pa == media.placeholder_ids(media.Image(b"cat", None), 4)
    assert set(pa).isdisjoint(media.placeholder_ids(b, 4))
    ids = media.expand([1, 99, 2, 99], 99, [a, b], 4)
    assert len(ids) == 10 and ids[1:5] == pa
    with pytest.raises(ValueError):
        media.expand([99], 99, [], 4)
    t = torch.tensor(ids)
    emb = torch.zeros(10, 8)
    out = media.splice_embeddings(t, emb, torch.ones(8, 8))
    assert out[1:5].sum() == 32 and out[0].sum() == 0
    img = media.Image.from_data_url("data:image/png;base64,Y2F0")
    assert img.data == b"cat"


@pytest.mark.gpu
def test_encoder_gpu_matches_cpu():
    cpu, gpu = VisionEncoder(CFG, "cpu"), VisionEncoder(CFG, "cuda")
    px = torch.randn(2, 3, 64, 64, generator=torch.Generator().manual_seed(1))
    a, b = cpu.encode(px).float(), gpu.encode(px).float().cpu()
    assert float((a - b).abs().max() / a.abs().max()) < 5e-2


def test_images_reach_the_model_through_the_engine():
    """An image in a prompt: the placeholder span takes the vision encoder's rows at prefill (also when the span is
    cut by chunked prefill), a different image changes the output, and the same image again hits the prefix cache."""
    import io

    from PIL import Image as PilImage

    from hibana_b200.api import media as api_media
    from hibana_b200.engine.executor import Executor
    from hibana_b200.engine.request import Request, SamplingParams
    from hibana_b200.models.hybrid import HybridModel
    from hibana_b200.target import get_target, scaled
    from hibana_b200.tokenizer import ByteTokenizer

    def png(color):
        buf = io.BytesIO()
        PilImage.new("RGB", (40, 30), color).save(buf, format="PNG")
        return buf.getvalue()

    t = scaled(get_target("tiny"), mtp_layers=0, vision=(64, 16, 64, 1, 2, 128), weight_format="bf16")
    model = HybridModel(t, "cpu", seed=0)
    assert model.vision_cfg.tokens_per_image == 4 and model.vision is not None
    tok = ByteTokenizer()

    def request(data, budget_text="describe: "):
        plan = api_media.MediaPlan([media.Image(data, None)])
        ids = api_media.expand(budget_text + api_media.MARKER + " please", tok, plan, 4)
        return Request(prompt_ids=ids, params=SamplingParams(max_tokens=3), media=plan)

    ex = Executor(model, max_batch=2, max_ctx=128, use_graphs=False)
    red = ex.generate_batch_requests([request(png("red"))])[0].output_ids
    again = request(png("red"))
    # the image span (negative, content-derived ids) is part of the cached prefix of the first request
    assert ex.state.cache.match(again.prompt_ids[:-1], split=False).length >= 14
    red2 = ex.generate_batch_requests([again])[0].output_ids
    assert red2 == red
    ex2 = Executor(model, max_batch=2, max_ctx=128, use_graphs=False)
    chunked = ex2.generate_batch_requests([request(png("red"))], prefill_budget=12)[0].output_ids   # cuts the span
    assert chunked == red
    blue = Executor(model, max_batch=2, max_ctx=128, use_graphs=False).generate_batch_requests(
        [request(png("blue"))])[0]
    assert any(i < 0 for i in blue.prompt_ids)
    emb_red = ex._vision_cache.embeddings(media.Image(png("red"), None))
    emb_blue = ex._vision_cache.embeddings(media.Image(png("blue"), None))
    assert emb_red.shape == (4, t.hidden) and not torch.equal(emb_red, emb_blue)
    with pytest.raises(ValueError):
        media.decode_pixels(media.Image(b"not an image", None), 64)
