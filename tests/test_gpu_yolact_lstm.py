"""GPU parity for C5 (YOLACT-style mask assembly) and C4 (imperative LSTM) against the TorchScript CPU oracle."""
import pytest
import torch

from oracle import workloads as W
from tests.util import close

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def fb(cuda_device):
    import functs_b200
    return functs_b200


def yolact_case(fb, proto, coef, boxes):
    masks, logits = fb.ops.yolact_masks(proto.cuda(), coef.cuda(), boxes.cuda(), with_logits=True)
    masks_fast = fb.ops.yolact_masks(proto.cuda(), coef.cuda(), boxes.cuda())
    assert torch.equal(masks, masks_fast)  # the value-check variant and the product variant agree bit for bit
    masks, logits = masks.cpu(), logits.cpu().permute(0, 2, 3, 1)  # [B,H,W,N]
    oracle = torch.jit.script(W.YolactMasks())
    ndiff = 0
    for s in range(0, proto.size(0), 16):  # the comparison runs in slices of 16 images to bound host memory
        e = min(s + 16, proto.size(0))
        ndiff += yolact_compare(oracle, proto[s:e], coef[s:e], boxes[s:e], masks[s:e], logits[s:e])
    print(f"mask bytes differing from the oracle inside the 1e-5 boundary band: {ndiff} of {masks.numel()}")
    return ndiff


def yolact_compare(oracle, proto, coef, boxes, masks, logits):
    want_masks, want_logits = oracle(proto, coef, boxes)
    # a dot product is accurate relative to the sum of the magnitudes of its terms
    mag = torch.einsum("bhwk,bnk->bhwn", proto.abs(), coef.abs())
    close(logits, want_logits, rtol=1e-5, scale=mag, what="mask logits")
    # thresholded masks: identical except where the fp64 logit is within 1e-5 of zero (the sigmoid > 0.5 boundary)
    diff = masks != want_masks
    ndiff = int(diff.sum())
    if ndiff:
        l64 = torch.einsum("bhwk,bnk->bnhw", proto.double(), coef.double())
        assert bool((l64[diff].abs() < 1e-5).all()), "mask mismatch away from the threshold boundary"
    return ndiff


def test_yolact_config_shapes(fb):
    proto, coef, boxes = W.make_yolact_inputs(2)
    yolact_case(fb, proto, coef, boxes)


def test_yolact_full_batch_against_oracle(fb):
    """B = 64 (the configured maximum): 122 M mask bytes against the oracle's own run."""
    proto, coef, boxes = W.make_yolact_inputs(64)
    yolact_case(fb, proto, coef, boxes)


def test_yolact_small_and_degenerate_boxes(fb):
    proto, coef, boxes = W.make_yolact_inputs(2, size=20, num_det=7)
    boxes[0, 0] = torch.tensor([5.0, 5.0, 5.0, 5.0])          # empty box -> still padded by 1
    boxes[0, 1] = torch.tensor([-4.0, -4.0, 30.0, 30.0])      # outside the image on every side
    boxes[0, 2] = torch.tensor([15.0, 3.0, 2.0, 12.0])        # x1 > x2
    boxes[1, 0] = torch.tensor([0.0, 0.0, 0.0, 20.0])
    yolact_case(fb, proto, coef, boxes)


def test_yolact_crop_golden(fb):
    """Crop rule against the fixture written by the reference's crop(): with all-ones coefficients on a one-hot
    prototype the logit is large and positive everywhere, so the mask is exactly the crop region."""
    import os
    f = torch.load(os.path.join(os.path.dirname(__file__), "golden", "yolact_crop.pt"))
    h, w, n = f["masks"].shape
    proto = torch.zeros(1, h, w, 32)
    proto[..., 0] = 10.0
    coef = torch.zeros(1, n, 32)
    coef[..., 0] = 1.0
    masks = fb.ops.yolact_masks(proto.cuda(), coef.cuda(), f["boxes"][None].cuda())
    want = (f["out"] > 0).permute(2, 0, 1).to(torch.uint8)
    assert torch.equal(masks[0].cpu(), want)


def test_yolact_full_batch_properties(fb):
    """B = 64: shard invariance and crop containment instead of an oracle run."""
    proto, coef, boxes = [t.cuda() for t in W.make_yolact_inputs(64)]
    full = fb.ops.yolact_masks(proto, coef, boxes)
    part = fb.ops.yolact_masks(proto[40:44].contiguous(), coef[40:44].contiguous(), boxes[40:44].contiguous())
    assert torch.equal(full[40:44], part)
    bounds = torch.stack([W.crop_bounds(b.cpu(), 138, 138) for b in boxes[:4]])  # [4,N,4]
    xs = torch.arange(138)
    inside = ((xs[None, None, None, :] >= bounds[:, :, 0, None, None]) & (xs[None, None, None, :] < bounds[:, :, 1, None, None]) &
              (xs[None, None, :, None] >= bounds[:, :, 2, None, None]) & (xs[None, None, :, None] < bounds[:, :, 3, None, None]))
    assert not bool((full[:4].cpu().bool() & ~inside).any())
    assert set(full.unique().tolist()) <= {0, 1}


# ---- LSTM ----------------------------------------------------------------------------------------------


def lstm_case(fb, seq, batch, hidden, mode):
    """Bar for fp32 values: 1e-5 relative.  h = o * tanh(c) lies in (-1, 1) and passes through zero, so a value is
    measured against max(|want|, 1): 1 is the bound of the gate activations every h and c is formed from.  No absolute
    term.  On top of that the device result is compared with the fp64 evaluation of the same program: the fp32 CUDA-core
    path (mode 1) must be as close to it as the fp32 CPU oracle itself is (factor 2); the tensor-core paths (modes 0, 2, 3)
    splits every fp32 operand into two TF32 numbers, which carry 22 of the 24 mantissa bits, so its products are about
    four times less accurate than fp32 products: factor 10, and always below 1e-5."""
    x, w_ih, w_hh, b_ih, b_hh = W.make_lstm_inputs(seq, batch, hidden)
    want_hs, want_cs = torch.jit.script(W.LSTMSeq(w_ih, w_hh, b_ih, b_hh))(x)
    mod = fb.workloads.LSTM(w_ih, w_hh, b_ih, b_hh)
    hs, cs = mod(x, mode=mode)
    assert mod.kernels_last_call == fb.workloads.LSTM.expected_launches(seq, batch, hidden, mode)
    o64 = W.LSTMSeq(w_ih.double(), w_hh.double(), b_ih.double(), b_hh.double())
    hs64, cs64 = o64(x.double())
    for name, got, want, truth in (("hs", hs, want_hs, hs64), ("cs", cs, want_cs, cs64)):
        e_or = float((want.double() - truth).abs().max())
        e_gpu = float((got.cpu().double() - truth).abs().max())
        print(f"T={seq} B={batch} H={hidden} mode={mode} {name}: max |v - v64| oracle {e_or:.2e}, gpu {e_gpu:.2e}")
        assert e_gpu <= (2.0 if mode == 1 else 10.0) * e_or + 1e-7 and e_gpu < 1e-5, (name, e_gpu, e_or)
        close(got.cpu(), want, rtol=1e-5, atol=0.0, scale=1.0, what=name)


def test_lstm_tensor_core_projection_matches_cuda_cores(fb):
    """Runs first among the LSTM tests: the tcgen05 (3xTF32) input projection against the fp32 CUDA-core projection on
    a small shape.  Agreement to 1e-5 is the evidence that the shared-memory descriptor strides describe the pre-tiled
    operand layout."""
    x, w_ih, w_hh, b_ih, b_hh = W.make_lstm_inputs(2, 64, 512)
    mod = fb.workloads.LSTM(w_ih, w_hh, b_ih, b_hh)
    ref_hs, _ = mod(x, mode=1)
    ref_hs = ref_hs.clone()
    hs, _ = mod(x, mode=0)
    err = float((hs - ref_hs).abs().max())
    print(f"tcgen05 projection vs CUDA-core projection, max |dh|: {err:.3e}")
    assert err < 1e-5


@pytest.mark.parametrize("mode", [1, 0, 2, 3])
def test_lstm_config_shapes(fb, mode):
    lstm_case(fb, 64, 64, 512, mode)


def test_lstm_tensor_core_recurrence_small(fb):
    """The tcgen05 recurrence (mode 2) on other lengths and on H = 256; a batch other than 64 takes the CUDA-core
    recurrence under the same mode."""
    lstm_case(fb, 1, 64, 512, 2)
    lstm_case(fb, 2, 64, 512, 2)
    lstm_case(fb, 9, 64, 256, 2)
    lstm_case(fb, 3, 33, 512, 2)


@pytest.mark.parametrize("seq,batch,hidden", [(3, 5, 256), (1, 64, 512), (7, 33, 512), (5, 8, 256)])
def test_lstm_ragged(fb, seq, batch, hidden):
    lstm_case(fb, seq, batch, hidden, 1)
    lstm_case(fb, seq, batch, hidden, 0)


def test_lstm_cell_golden(fb):
    """One step against the fixture written by the reference's LSTMCell.forward needs H in {256, 512}; the fixture
    is H=32, so embed it: zero-pad weights to H=256 (extra units stay decoupled) and compare the first 32 units."""
    import os
    f = torch.load(os.path.join(os.path.dirname(__file__), "golden", "lstm_cell.pt"))
    hid, big = 32, 256
    bat = f["x"].size(0)
    w_ih = torch.zeros(4, big, big)
    w_hh = torch.zeros(4, big, big)
    b_ih = torch.zeros(4, 1, big)
    b_hh = torch.zeros(4, 1, big)
    w_ih[:, :hid, :hid] = f["w_ih"]
    w_hh[:, :hid, :hid] = f["w_hh"]
    b_ih[..., :hid] = f["b_ih"]
    b_hh[..., :hid] = f["b_hh"]
    # the fixture starts from non-zero (h0, c0); the kernel starts from zero, so check the zero-state step of the
    # same cell with the oracle, which the CPU test pins to the fixture
    x = torch.zeros(1, bat, big)
    x[0, :, :hid] = f["x"]
    want_h, want_c = W.lstm_cell(x[0], torch.zeros(bat, big), torch.zeros(bat, big), w_ih, w_hh, b_ih, b_hh)
    hs, cs = fb.workloads.LSTM(w_ih, w_hh, b_ih, b_hh)(x, mode=1)
    close(hs[0].cpu(), want_h, rtol=1e-5, atol=1e-6, what="h1")
    close(cs[0].cpu(), want_c, rtol=1e-5, atol=1e-6, what="c1")


def test_lstm_rejects_unsupported_hidden(fb):
    x, w_ih, w_hh, b_ih, b_hh = W.make_lstm_inputs(2, 2, 64)
    with pytest.raises(fb.FunctsB200Error):
        fb.workloads.LSTM(w_ih, w_hh, b_ih, b_hh)(x)
