"""Generate ``kv_layout_inference.json`` by running the reference's own layout inference.

Run where the reference checkout is available (``PEGAFLOW_REFERENCE``, default: a ``reference``
directory beside this repository).  The reference's pure-Python ``_infer_kv_cache_registration``
(python/pegaflow/connector/worker.py:65-151) is imported with the native extension stubbed
out by the reference's own ``unit_stubs`` helper, and evaluated on a grid of tensor
shapes/strides.  The output is committed so the tests never need the reference at run time.
"""
import itertools
import json
import os
import sys

_REPO = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
REF = os.environ.get("PEGAFLOW_REFERENCE", os.path.join(os.path.dirname(_REPO), "reference"))
sys.path.insert(0, os.path.join(REF, "python"))
from tests.unit_stubs import install_connector_unit_stubs  # noqa: E402

install_connector_unit_stubs()
from pegaflow.connector.worker import _infer_kv_cache_registration  # noqa: E402


class FakeTensor:
    def __init__(self, shape, stride, element_size):
        self.shape, self._stride, self._es = tuple(shape), tuple(stride), element_size

    def stride(self):
        return self._stride

    def element_size(self):
        return self._es


def contiguous(shape):
    st, acc = [], 1
    for d in reversed(shape):
        st.append(acc)
        acc *= d
    return tuple(reversed(st))


def permuted(shape, perm):
    """Strides of a tensor whose memory order is ``perm`` of the logical dims."""
    mem_shape = [shape[p] for p in perm]
    mem_stride = contiguous(mem_shape)
    out = [0] * len(shape)
    for pos, p in enumerate(perm):
        out[p] = mem_stride[pos]
    return tuple(out)


cases = []


def add(shape, stride, es, logical, is_mla=False, is_recurrent_state=False):
    rec = dict(shape=list(shape), stride=list(stride), element_size=es, logical_block_size=logical, is_mla=is_mla,
               is_recurrent_state=is_recurrent_state)
    try:
        info = _infer_kv_cache_registration(FakeTensor(shape, stride, es), logical, is_mla=is_mla,
                                            is_recurrent_state=is_recurrent_state)
        rec["result"] = dict(layout=info.layout, num_blocks=info.num_blocks, bytes_per_block=info.bytes_per_block,
                             kv_stride_bytes=info.kv_stride_bytes, segments=info.segments,
                             physical_blocks_per_logical_block=info.physical_blocks_per_logical_block)
    except ValueError as e:
        rec["error"] = str(e)
    cases.append(rec)


# FlashAttention form (2, num_blocks, block, heads, dim), NHD and HND memory orders
for nb, blk, h, d, es in itertools.product([6, 256, 8192], [16, 64], [1, 2, 8], [64, 128], [1, 2]):
    shp = (2, nb, blk, h, d)
    add(shp, contiguous(shp), es, blk)
    add(shp, permuted(shp, (0, 1, 3, 2, 4)), es, blk)          # HND inside a block
    add(shp, permuted(shp, (1, 0, 2, 3, 4)), es, blk)          # (num_blocks, 2, ...) memory: interleaved K/V
# FlashInfer form (num_blocks, 2, block, heads, dim)
for nb, blk, h, d in itertools.product([6, 256], [16, 32], [2, 8], [128]):
    shp = (nb, 2, blk, h, d)
    add(shp, contiguous(shp), 2, blk)
# separate K or V tensor [num_blocks, block, heads, dim]
for nb, h in itertools.product([256, 8192], [1, 2, 8]):
    shp = (nb, 16, h, 128)
    add(shp, contiguous(shp), 2, 16)
    add(shp, permuted(shp, (0, 2, 1, 3)), 2, 16)
# cross-layer fused buffer (num_blocks, layers, 2, block, heads, dim)
for nb, layers in itertools.product([6, 64], [28, 32, 93]):
    shp = (nb, layers, 2, 64, 1, 128)
    add(shp, contiguous(shp), 2, 128)
# MLA latent (num_blocks, block, 576) with logical/physical grouping
for nb, blk, logical, es in itertools.product([0, 1, 2, 5, 6, 256], [0, 64, 96, 128], [0, 64, 128, 256], [1, 2]):
    shp = (nb, blk, 576)
    add(shp, contiguous(shp), es, logical, is_mla=True)
add((3, 128, 576), (0, 576, 1), 2, 128, is_mla=True)
add((2, 64, 576), (64 * 576, 576, 1), 2, 128, is_mla=True)
# recurrent state pages
add((2, 1, 4096), (4096, 4096, 1), 2, 1536, is_mla=True, is_recurrent_state=True)
add((2, 1, 4096), (4096, 4096, 1), 2, 1536, is_mla=False, is_recurrent_state=True)
add((16, 8, 512), contiguous((16, 8, 512)), 4, 16, is_recurrent_state=True)

out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "kv_layout_inference.json")
with open(out, "w") as f:
    json.dump(dict(source="python/pegaflow/connector/worker.py:65-151 (_infer_kv_cache_registration)", cases=cases),
              f, indent=0, separators=(",", ":"))
print(f"wrote {len(cases)} cases to {out}")
