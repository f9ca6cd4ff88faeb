"""FP8 checkpoint ingestion (CPU): scale layouts of community checkpoints are mapped onto
weight_scale [N, K/G] without changing a code, through a state dict and through safetensors files."""
import pytest
import torch
import torch.nn as nn

from tfp8 import FP8Linear
from tfp8.checkpoint import linear_from_checkpoint, load_fp8_state_dict, load_safetensors, normalize_scale
from tfp8.quantize import dequantize_weight


def _block_quantize(w, bn, bk):
    """Reference block quantizer of the test: one float32 scale per bn x bk block, E4M3FN codes."""
    N, K = w.shape
    rows, cols = -(-N // bn), -(-K // bk)
    scale = torch.empty(rows, cols)
    q = torch.empty(N, K, dtype=torch.float8_e4m3fn)
    for i in range(rows):
        for j in range(cols):
            blk = w[i * bn:(i + 1) * bn, j * bk:(j + 1) * bk]
            s = float(blk.abs().max()) / 448.0 or 1.0
            scale[i, j] = s
            q[i * bn:(i + 1) * bn, j * bk:(j + 1) * bk] = (blk / s).clamp(-448, 448).to(torch.float8_e4m3fn)
    return q, scale


def test_scale_layouts():
    N, K = 6, 256
    s, G = normalize_scale(torch.tensor(0.5), N, K)
    assert s.shape == (N, 1) and G == K and bool((s == 0.5).all())
    s, G = normalize_scale(torch.arange(1.0, N + 1), N, K)
    assert s.shape == (N, 1) and G == K and s[3, 0] == 4.0
    s, G = normalize_scale(torch.rand(N, 4), N, K)
    assert s.shape == (N, 4) and G == 64
    blocks = torch.tensor([[1.0, 2.0], [3.0, 4.0]])                  # 4 x 128 blocks of a 6 x 256 weight
    s, G = normalize_scale(blocks, N, K, block=(4, 128))
    assert G == 128 and s.shape == (N, 2)
    assert s[:4].tolist() == [[1.0, 2.0]] * 4 and s[4:].tolist() == [[3.0, 4.0]] * 2
    s, G = normalize_scale(torch.rand(3, 2), N, K)                    # block sizes follow from the shapes
    assert G == 128 and s.shape == (N, 2)
    with pytest.raises(ValueError):
        normalize_scale(torch.rand(4, 3), N, K)                        # does not tile
    with pytest.raises(ValueError):
        normalize_scale(torch.rand(5), N, K)


def test_block_scaled_checkpoint_round_trip():
    torch.manual_seed(0)
    w = torch.randn(200, 384) * 0.05
    q, scale = _block_quantize(w, 128, 128)
    layer = linear_from_checkpoint(q, scale, bias=torch.randn(200), fmt="e4m3fn", block=(128, 128))
    assert isinstance(layer, FP8Linear) and layer.group_size == 128
    assert torch.equal(layer.qweight, q.view(torch.uint8))            # codes adopted verbatim
    want = q.float() * scale.repeat_interleave(128, 0)[:200].repeat_interleave(128, 1)
    assert torch.equal(dequantize_weight(layer.qweight, layer.weight_scale, "e4m3fn", 128), want)
    x = torch.randn(3, 384)
    layer.out_dtype = torch.float32
    assert torch.allclose(layer(x), x @ want.T + layer.bias_f32, rtol=1e-5, atol=1e-5)


class _Net(nn.Module):
    def __init__(self):
        super().__init__()
        self.embed = nn.Embedding(50, 256)
        self.proj = nn.Linear(256, 384, bias=False)
        self.norm = nn.LayerNorm(384)
        self.head = nn.Linear(384, 50)                                 # stays full precision in the checkpoint

    def forward(self, t):
        return self.head(self.norm(self.proj(self.embed(t))))


def _checkpoint():
    torch.manual_seed(1)
    ref = _Net()
    q, scale = _block_quantize(ref.proj.weight.data, 128, 128)
    tensors = {k: v.clone() for k, v in ref.state_dict().items() if k != "proj.weight"}
    tensors["proj.weight"] = q
    tensors["proj.weight_scale_inv"] = scale
    with torch.no_grad():
        ref.proj.weight.copy_(q.float() * scale.repeat_interleave(128, 0).repeat_interleave(128, 1))
    return ref, tensors


def test_state_dict_and_safetensors(tmp_path):
    ref, tensors = _checkpoint()
    t = torch.randint(0, 50, (2, 7))
    want = ref(t)
    net = _Net()
    assert load_fp8_state_dict(net, tensors) == ["proj"]
    assert isinstance(net.proj, FP8Linear) and isinstance(net.head, nn.Linear)
    net.proj.out_dtype = torch.float32
    assert torch.allclose(net(t), want, rtol=1e-4, atol=1e-4)
    # the same through a sharded safetensors checkpoint
    from safetensors.torch import save_file
    names = sorted(tensors)
    save_file({k: tensors[k].contiguous() for k in names[:3]}, str(tmp_path / "a.safetensors"))
    save_file({k: tensors[k].contiguous() for k in names[3:]}, str(tmp_path / "b.safetensors"))
    net2 = _Net()
    assert load_safetensors(net2, [tmp_path / "a.safetensors", tmp_path / "b.safetensors"]) == ["proj"]
    net2.proj.out_dtype = torch.float32
    assert torch.allclose(net2(t), want, rtol=1e-4, atol=1e-4)
    # strict: an FP8 weight without its scale is an error, a stray tensor too
    broken = {k: v for k, v in tensors.items() if k != "proj.weight_scale_inv"}
    with pytest.raises(KeyError):
        load_fp8_state_dict(_Net(), broken)
    with pytest.raises(KeyError):
        load_fp8_state_dict(_Net(), dict(tensors, stray=torch.zeros(1)))
