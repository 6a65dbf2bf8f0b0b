"""turboloader_b200: a B200 (sm_100a) implementation of TurboLoader's fused image-transform
hot path -- crop, horizontal flip, bilinear resize, mean/std normalize, HWC->NCHW/NHWC and
fp32/bf16 cast of pre-decoded uint8 images in one kernel launch per batch -- behind the
names of TurboLoader's own GPU operators and resident loader.

The compute path is the C-ABI shared library built from ``csrc/`` (see ``include/``);
there is no CPU fallback: operators raise if the library or an sm_100 device is missing.
"""
from .ops import (IMAGENET_MEAN, IMAGENET_STD, cuda_available, cuda_crop_resize_normalize, cuda_device_name,
                  cuda_normalize_resident, cuda_normalize_resident_gather, cuda_resize_normalize,
                  cuda_resize_normalize_from_device, features,
                  fused_plan, fused_transform, launch_count, make_desc, cuda_video_clip_yuv420,
                  cuda_video_yuv420_batch, video_yuv420)
from .cuda_loader import CudaResidentLoader, _CudaArray
from .stream_loader import CudaStreamLoader
from .direct_loader import DirectBatchLoader
from .dataloader import DataLoader, ImageNetNormalize
from .augment import pick_crops
from .sharding import (CONTIGUOUS, HASH_BASED, INTERLEAVED, DistributedSampler, ShardingCoordinator,
                       ShardingStrategy, direct_order, shard_indices)

__version__ = "0.1.0"
__all__ = [
    "IMAGENET_MEAN", "IMAGENET_STD", "cuda_available", "cuda_device_name", "cuda_resize_normalize",
    "cuda_crop_resize_normalize", "cuda_normalize_resident", "cuda_normalize_resident_gather",
    "cuda_resize_normalize_from_device",
    "fused_transform", "fused_plan", "make_desc", "features", "launch_count", "cuda_video_yuv420_batch", "cuda_video_clip_yuv420", "video_yuv420",
    "CudaResidentLoader", "CudaStreamLoader", "_CudaArray",
    "DataLoader", "DirectBatchLoader", "ImageNetNormalize", "pick_crops",
    "ShardingStrategy", "ShardingCoordinator", "DistributedSampler", "direct_order", "shard_indices",
    "CONTIGUOUS", "INTERLEAVED", "HASH_BASED",
]
