"""TEST INFRASTRUCTURE ONLY: drive upstream's own preprocessor (compiled unmodified into
oracle/_ref/ by `make -C oracle ref_search`) the way ROF_evaluation/ROF_main.py:71-127 does,
and return every index array it produces.  Used to pin the product's own search and plan
builder bit-for-bit and to generate the fixtures under tests/golden/."""
import contextlib
import importlib.util
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def load_module():
    ref_dir = os.path.join(HERE, "_ref")
    for f in sorted(os.listdir(ref_dir)) if os.path.isdir(ref_dir) else []:
        if f.startswith("reuse_search_ext") and f.endswith(".so"):
            spec = importlib.util.spec_from_file_location("reuse_search_ext", os.path.join(ref_dir, f))
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            return mod
    return None


@contextlib.contextmanager
def _quiet():
    """upstream prints progress with std::cout; silence fd 1 for the duration of a call"""
    sys.stdout.flush()
    saved = os.dup(1)
    devnull = os.open(os.devnull, os.O_WRONLY)
    os.dup2(devnull, 1)
    try:
        yield
    finally:
        os.dup2(saved, 1)
        os.close(saved)
        os.close(devnull)


def run(indptr_dst, indices_src, indptr_src, indices_dst, part_size, mod=None):
    """ROF_main.py:71-127 with discard_remainder_part=True.  Needs at least 9 nodes: upstream's
    split_part prints indptr_dst[0..9] unconditionally (reuse_search_ext.h:89-94)."""
    mod = mod or load_module()
    if mod is None:
        raise RuntimeError("oracle/_ref/reuse_search_ext*.so not built")
    u32 = lambda a: np.ascontiguousarray(a, dtype=np.uint32)
    indptr_dst, indices_src, indptr_src, indices_dst = map(u32, (indptr_dst, indices_src, indptr_src, indices_dst))
    assert indptr_dst.shape[0] >= 10
    a = np.empty(0, dtype=np.uint32)
    b = np.empty(0, dtype=np.uint32)
    with _quiet():
        part_ptr, part2Node, acc = mod.py_split_part(a, b, indptr_dst, part_size)
        lists, nums = mod.py_get_part_intersect(part_ptr, indices_src, indptr_src, indices_dst, part_size, True)
        index_ordered, index_picked = mod.py_greedy_max_reuse(nums, part_ptr, indices_src)
        new_indices_src, _, part_pointers_cache, column_index_cache, part_cache_flagindex = \
            mod.py_reorganize_indices(part_ptr, indices_src, lists, index_picked, indptr_dst, acc, part_size)
        uniq_col, uniq_ptr, p2n_ptr, p2n_col = mod.py_reorganize_indices_uniquely(
            part_ptr, indices_src, lists, index_picked, indptr_dst, acc, part_size)
    i32 = lambda a: np.asarray(a).astype(np.int32)
    return {
        "part_size": int(part_size),
        "part_pointers": i32(part_ptr), "part2Node": i32(part2Node), "num_parts_per_node_acc": i32(acc),
        "intersection_num_per_part": i32(nums[0]),
        "index_picked": i32(index_picked),
        "picked_fanout": i32(nums[0])[i32(index_picked)] if len(index_picked) else np.zeros(0, np.int32),
        "column_index": i32(new_indices_src),
        "part_pointers_cache": i32(part_pointers_cache), "column_index_cache": i32(column_index_cache),
        "part_cache_flagindex": i32(part_cache_flagindex),
        "uniqpart_column_index": i32(uniq_col), "uniqpart_pointers": i32(uniq_ptr),
        "part2Node_ptr": i32(p2n_ptr), "part2Node_col": i32(p2n_col),
        "original_column_index": i32(indices_src),
    }
