"""Named operations for ``loop-explore --op-name`` / ``--op-name-list``.

The reference keeps this registry in ``artifacts/operations.py:8-70`` and fills it from its
benchmark size tables (``artifacts/register_ttile_operations.py:17-46`` over
``schedules/ttile/prob_sizes.py``: Yolo9000, MobilNet, ResNet18 convolution layers and the
LLM / Polybench matmul shapes; ``artifacts/register_subgraph_operations.py:10-36`` over
``artifacts/subgraph_sizes.py``: SqueezeNet and AlexNet).  The same names and sizes are
served here, so ``--op-name ResNet18_02`` means the same layer on either side, plus this
backend's own benchmark shapes (c1 .. c5).

An entry has ``dims`` (loop extents, the operator's dimension names) and ``params``
(``SH`` / ``SW``, the convolution strides); the driver takes the values of both in order
(``search/explore.py:836-840``).  For convolutions ``h`` and ``w`` are OUTPUT rows and
columns: the input is ``h * SH + r - 1`` by ``w * SW + s - 1`` (``search/explore.py:239-258``).
"""

from __future__ import annotations

import itertools
import logging

logger = logging.getLogger(__name__)

_REGISTRY: dict[str, dict[str, dict]] = {}


def register_operation(operator: str, name: str, dims: dict[str, int],
                       params: dict[str, int] | None = None) -> None:
    ops = _REGISTRY.setdefault(operator, {})
    if name.lower() in ops:
        logger.warning("operation %s/%s is already registered", operator, name.lower())
    ops[name.lower()] = {"name": name, "dims": dict(dims), "params": dict(params or {})}


def get_operation(operator: str, name: str) -> dict:
    if operator not in _REGISTRY:
        raise ValueError(f"operator {operator} not registered in operation registry")
    try:
        return _REGISTRY[operator][name.lower()]
    except KeyError:
        raise ValueError(
            f"operation name {name} for operator {operator} not registered in operation registry") from None


def has_operation(operator: str, name: str) -> bool:
    return name.lower() in _REGISTRY.get(operator, {})


def list_operations(operator: str = "") -> list[tuple[str, str]]:
    if operator == "":
        return list(itertools.chain(*[list_operations(o) for o in _REGISTRY]))
    if operator not in _REGISTRY:
        raise ValueError(f"operator {operator} not registered in operation registry")
    return [(operator, e["name"]) for e in _REGISTRY[operator].values()]


def operation_dims(operator: str, name: str) -> list[int]:
    """Values of dims then params, the order the operator's graph builder takes."""
    op = get_operation(operator, name)
    return [*op["dims"].values(), *op["params"].values()]


# name: (n, h, w, f, r, s, c, SH, SW) -- h, w are OUTPUT rows and columns
CONV2D_LAYERS = {
    "Yolo9000_00": (1, 544, 544, 32, 3, 3, 3, 1, 1),
    "Yolo9000_02": (1, 272, 272, 64, 3, 3, 32, 1, 1),
    "Yolo9000_04": (1, 136, 136, 128, 3, 3, 64, 1, 1),
    "Yolo9000_05": (1, 136, 136, 64, 1, 1, 128, 1, 1),
    "Yolo9000_08": (1, 68, 68, 256, 3, 3, 128, 1, 1),
    "Yolo9000_09": (1, 68, 68, 128, 1, 1, 256, 1, 1),
    "Yolo9000_12": (1, 34, 34, 512, 3, 3, 256, 1, 1),
    "Yolo9000_13": (1, 34, 34, 256, 1, 1, 512, 1, 1),
    "Yolo9000_18": (1, 17, 17, 1024, 3, 3, 512, 1, 1),
    "Yolo9000_19": (1, 17, 17, 512, 1, 1, 1024, 1, 1),
    "Yolo9000_23": (1, 17, 17, 28272, 1, 1, 1024, 1, 1),
    "MobilNet_01": (1, 112, 112, 32, 3, 3, 32, 1, 1),
    "MobilNet_02": (1, 112, 112, 64, 3, 3, 64, 2, 2),
    "MobilNet_03": (1, 56, 56, 128, 3, 3, 128, 1, 1),
    "MobilNet_04": (1, 56, 56, 128, 3, 3, 128, 2, 2),
    "MobilNet_05": (1, 28, 28, 256, 3, 3, 256, 1, 1),
    "MobilNet_06": (1, 28, 28, 256, 3, 3, 256, 2, 2),
    "MobilNet_07": (1, 14, 14, 512, 3, 3, 512, 1, 1),
    "MobilNet_08": (1, 14, 14, 512, 3, 3, 512, 2, 2),
    "MobilNet_09": (1, 7, 7, 1024, 3, 3, 1024, 1, 1),
    "ResNet18_01": (1, 224, 224, 64, 7, 7, 3, 2, 2),
    "ResNet18_02": (1, 56, 56, 64, 3, 3, 64, 1, 1),
    "ResNet18_03": (1, 56, 56, 64, 1, 1, 64, 1, 1),
    "ResNet18_04": (1, 56, 56, 128, 3, 3, 64, 2, 2),
    "ResNet18_05": (1, 56, 56, 128, 1, 1, 64, 2, 2),
    "ResNet18_06": (1, 28, 28, 128, 3, 3, 128, 1, 1),
    "ResNet18_07": (1, 28, 28, 256, 3, 3, 128, 2, 2),
    "ResNet18_08": (1, 28, 28, 256, 3, 3, 128, 1, 1),
    "ResNet18_09": (1, 14, 14, 256, 3, 3, 256, 1, 1),
    "ResNet18_10": (1, 14, 14, 512, 3, 3, 512, 2, 2),
    "ResNet18_11": (1, 14, 14, 512, 1, 1, 256, 2, 2),
    "ResNet18_12": (1, 7, 7, 512, 3, 3, 512, 1, 1),
    "SqueezeNet_00": (1, 224, 224, 96, 7, 7, 3, 2, 2),
    "SqueezeNet_01": (1, 54, 54, 16, 1, 1, 96, 1, 1),
    "SqueezeNet_03": (1, 56, 56, 64, 3, 3, 16, 1, 1),
    "SqueezeNet_04": (1, 54, 54, 16, 1, 1, 128, 1, 1),
    "SqueezeNet_05": (1, 54, 54, 32, 1, 1, 128, 1, 1),
    "SqueezeNet_07": (1, 54, 54, 128, 3, 3, 32, 1, 1),
    "SqueezeNet_08": (1, 27, 27, 32, 1, 1, 256, 1, 1),
    "SqueezeNet_11": (1, 27, 27, 48, 1, 1, 256, 1, 1),
    "SqueezeNet_13": (1, 27, 27, 192, 3, 3, 48, 1, 1),
    "SqueezeNet_14": (1, 27, 27, 48, 1, 1, 384, 1, 1),
    "SqueezeNet_17": (1, 27, 27, 256, 3, 3, 64, 1, 1),
    "SqueezeNet_21": (1, 15, 15, 1000, 1, 1, 512, 1, 1),
    "AlexNet_00": (1, 228, 228, 64, 11, 11, 3, 4, 4),
    "AlexNet_01": (1, 31, 31, 192, 5, 5, 64, 1, 1),
    "AlexNet_02": (1, 15, 15, 384, 3, 3, 192, 1, 1),
    "AlexNet_03": (1, 15, 15, 256, 3, 3, 384, 1, 1),
    "AlexNet_04": (1, 15, 15, 256, 3, 3, 256, 1, 1),
}
# name: (i, j, k)
MATMUL_SIZES = {
    "Llama3AttMm": (8192, 8192, 4096),
    "Polybench_medium": (200, 224, 240),
    "Polybench_large": (1000, 1104, 1200),
    "Polybench_extralarge": (2000, 2304, 2600),
    "Llama3_In": (4096, 4096, 128),
    "Llama3_QK": (128, 4096, 8192),
    "Llama3_QKV": (128, 8192, 4096),
    "Llama3_FC": (4096, 4096, 4096),
    "Gemma27B_In": (4608, 4096, 256),
    "Gemma27B_QK": (256, 4608, 8192),
    "Gemma27B_QKV": (256, 8192, 4608),
    "Gemma27B_FC": (4608, 36864, 4608),
    "Gemma9B_In": (3584, 4096, 256),
    "Gemma9B_QK": (256, 3584, 8192),
    "Gemma9B_QKV": (256, 8192, 3584),
    "Gemma9B_FC": (3584, 14336, 3584),
    "Gemma7B_In": (3072, 4096, 256),
    "Gemma7B_QK": (256, 3072, 8192),
    "Gemma7B_QKV": (256, 8192, 3072),
    "Gemma7B_FC": (3072, 24576, 3072),
    "Gemma2B_In": (2048, 4096, 256),
    "Gemma2B_QK": (256, 2048, 8192),
    "Gemma2B_QKV": (256, 8192, 2048),
    "Gemma2B_FC": (2048, 16384, 2048),
    "AlexNet_FC6": (1, 4096, 9216),
    "AlexNet_FC7": (1, 4096, 4096),
    "AlexNet_FC8": (1, 1000, 4096),
}


def _register_all() -> None:
    for name, (n, h, w, f, r, s, c, sh, sw) in CONV2D_LAYERS.items():
        register_operation("conv2d", name, dict(n=n, h=h, w=w, f=f, r=r, s=s, c=c), dict(SH=sh, SW=sw))
    for name, (i, j, k) in MATMUL_SIZES.items():
        register_operation("matmul", name, dict(i=i, j=j, k=k))
    # this backend's benchmark configurations
    register_operation("matmul", "c1", dict(i=512, j=256, k=1024))
    register_operation("matmul_relu", "c2", dict(i=4096, j=4096, k=4096))
    register_operation("matmul", "c4_gemm", dict(i=8192, j=1024, k=8192))
    register_operation("matmul", "c5_shard8", dict(i=8192, j=8192, k=8192))
    register_operation("conv2d", "c3_conv", dict(n=32, h=56, w=56, f=64, r=3, s=3, c=64), dict(SH=1, SW=1))


_register_all()
