"""GPU tests of the streaming loader (dataset in pinned host memory, K-slot copy + kernel pipeline):
every batch is bit-identical to the CPU oracle on the same slice of the dataset, in index order."""
import numpy as np
import pytest

import turboloader_b200 as t
from oracle import oracle as O
from turboloader_b200 import synthetic as S

from helpers import check_bf16

pytestmark = pytest.mark.gpu
MEAN, STD = t.IMAGENET_MEAN, t.IMAGENET_STD


def _data(n=70, hw=20, seed=3):
    return np.random.RandomState(seed).randint(0, 256, size=(n, hw, hw, 3), dtype=np.uint8)


def _oracle(data, lo, hi, box=None, dst=None):
    flat, offsets, sizes = S.uniform_dataset(data)
    sel = np.arange(lo, hi, dtype=np.int64)
    boxes = None if box is None else np.tile(np.array([box], np.int32), (hi - lo, 1))
    h, w = data.shape[1:3]
    dh, dw = dst if dst else ((box[3], box[2]) if box else (h, w))
    return O.fused_batch(flat, offsets, sizes, sel, boxes, None, dh, dw, MEAN, STD, True)


@pytest.mark.parametrize("synchronize", [False, True])
@pytest.mark.parametrize("drop_last", [True, False])
def test_batches_in_index_order_match_the_oracle(synchronize, drop_last):
    import torch
    data = _data()
    dl = t.CudaStreamLoader.from_array(data, batch_size=16, slots=3, drop_last=drop_last, synchronize=synchronize)
    assert len(dl) == (4 if drop_last else 5)
    for epoch in range(2):  # the slots are reused across epochs
        got = [torch.as_tensor(b, device="cuda").clone() for b in dl]
        assert len(got) == len(dl)
        for i, b in enumerate(got):
            lo, hi = i * 16, min(70, i * 16 + 16)
            assert tuple(b.shape) == (hi - lo, 3, 20, 20)
            assert np.array_equal(b.cpu().numpy(), _oracle(data, lo, hi)), f"epoch {epoch} batch {i}"
    assert dl.device_status() == 0


def test_a_batch_stays_valid_while_the_next_ones_are_prefetched():
    """Without cloning: consume each batch on the current stream after asking for the next one."""
    import torch
    data = _data(n=96)
    dl = t.CudaStreamLoader.from_array(data, batch_size=8, slots=3)
    sums, prev = [], None
    for b in dl:
        cur = torch.as_tensor(b, device="cuda")
        if prev is not None:
            sums.append(prev.double().sum())  # uses batch i-1 after batch i was handed out
        prev = cur
    sums.append(prev.double().sum())
    torch.cuda.synchronize()
    for i, s in enumerate(sums):
        want = _oracle(data, i * 8, i * 8 + 8).astype(np.float64).sum()
        assert abs(float(s) - want) < 1e-6 * max(1.0, abs(want))


def test_centre_crop_resize_bf16_channels_last():
    import torch
    data = _data(n=40, hw=32, seed=9)
    dl = t.CudaStreamLoader.from_array(data, batch_size=16, crop_size=28, output_size=24, dtype=torch.bfloat16,
                                      channels_last=True, drop_last=False, slots=4)
    outs = [b.clone() for b in dl]
    assert [o.shape[0] for o in outs] == [16, 16, 8]
    for i, b in enumerate(outs):
        assert b.dtype == torch.bfloat16 and tuple(b.shape[1:]) == (24, 24, 3)
        lo, hi = i * 16, min(40, i * 16 + 16)
        want = O.nchw_to_nhwc(_oracle(data, lo, hi, box=(2, 2, 28, 28), dst=(24, 24)))
        assert check_bf16(b.view(torch.int16).cpu().numpy().view(np.uint16), O.bf16_bits(want)) == 0


def test_invalid_arguments():
    with pytest.raises(ValueError):
        t.CudaStreamLoader.from_array(np.zeros((4, 8, 8), np.uint8))
    with pytest.raises(RuntimeError):
        t.CudaStreamLoader.from_array(np.zeros((4, 8, 8, 3), np.uint8), crop_size=12)  # crop leaves the image
