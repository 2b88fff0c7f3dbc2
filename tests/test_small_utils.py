"""Adapter switching and tensor → image previews."""
import pytest
import torch


def test_switch_adapter_restores_and_validates():
    from unirl_b200.models.qwen3.modeling import Qwen3Config, Qwen3Transformer
    from unirl_b200.train import inject
    from unirl_b200.utils.adapter_utils import adapter_names, switch_adapter

    model = Qwen3Transformer(Qwen3Config.tiny(num_hidden_layers=1), dtype=torch.float32).init_weights(0)
    with switch_adapter(model, "anything"):  # no adapters: passes through
        pass
    inject.inject_nft(model, rank=2, alpha=4.0, target_modules=("q_proj", "v_proj"))
    assert adapter_names(model) == ["default", "old"]
    hosts = [m for m in model.modules() if hasattr(m, "lora")]
    assert hosts and all(getattr(m, "_lora_active", "default") == "default" for m in hosts)
    with pytest.raises(RuntimeError):
        with switch_adapter(model, "old"):
            assert all(m._lora_active == "old" for m in hosts)
            raise RuntimeError("inside")
    assert all(m._lora_active == "default" for m in hosts)
    with pytest.raises(KeyError):
        with switch_adapter(model, "missing"):
            pass


def test_tensor_previews():
    from unirl_b200.utils.media import tensor_frame_to_pil, tensor_to_pil

    img = tensor_frame_to_pil(torch.tensor([[[0.0, 0.5], [1.0, 2.0]]]))  # one channel, one value out of range
    assert img.mode == "RGB" and img.size == (2, 2) and img.getpixel((1, 1)) == (255, 255, 255) and img.getpixel((1, 0)) == (128, 128, 128)
    vids = torch.zeros(2, 3, 5, 4, 6)
    vids[:, :, 2] = 1.0
    previews = tensor_to_pil(vids)
    assert len(previews) == 2 and previews[0].size == (6, 4) and previews[0].getpixel((0, 0)) == (255, 255, 255)  # the middle frame
    with pytest.raises(ValueError):
        tensor_to_pil(torch.zeros(3, 4))
