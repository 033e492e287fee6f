"""Per-shape tile table: the counterpart of the reference's tuning logs.

The reference keeps, per (data shape, weight shape, strides), the index of the best of its
schedule candidates (``cpu-tune.log`` / ``gpu-tune.log``, loaded by
``python/tensorizer/tune.py:20-51``) and logs the shapes its models contain (``cpu-shapes.log``).
Here an entry overrides the library's tile heuristics for one convolution shape: the width of a
column block, the depth of a pipeline stage, sub-tiles per tile, the split-K limit
(``unit_tile_entry`` in ``include/unit_b200.h``).

* ``shape_corpus.json``  the int8 NCHW16c convolution shapes of the reference's ``cpu-shapes.log``
  (made by ``python -m unit_b200.tile_table corpus <cpu-shapes.log>``); shapes only, no data;
* ``tile_table.json``    entries found by ``python -m unit_b200.tune`` on a B200; loaded and handed
  to the library on first use of an operator (absent file: heuristics only).
"""
from __future__ import annotations

import ast
import ctypes
import json
import os
import sys
from typing import Dict, Iterable, List, Tuple

from . import _lib

_HERE = os.path.dirname(os.path.abspath(__file__))
CORPUS_PATH = os.path.join(_HERE, 'shape_corpus.json')
TABLE_PATH = os.path.join(_HERE, 'tile_table.json')
FIELDS = ('c_in', 'c_block', 'c_out', 'kh', 'kw', 'stride_h', 'stride_w', 'n', 'h', 'w', 'bn', 'kc', 'mt', 'ksplit')

_VERSION = 0   # bumped whenever the library's table changes: packed-weight caches key on it


def version() -> int:
    return _VERSION


def parse_shape_log(lines: Iterable[str]) -> List[dict]:
    """Unique int8 convolution shapes of a log in the reference's format,
    ``(n, c/cb, h, w, cb) (o/16, c/cb, kh, kw, cb/4, 16, 4) (sh, sw) ...``; dense rows and channel
    blocks other than 16 are skipped.  Spatial sizes in that log are pre-padded."""
    seen: Dict[tuple, int] = {}
    for line in lines:
        line = line.strip()
        if not line.startswith('(') or 'dense' in line:
            continue
        try:
            parts = []
            rest = line
            for _ in range(3):
                end = rest.index(')') + 1
                parts.append(ast.literal_eval(rest[:end]))
                rest = rest[end:].lstrip()
        except (ValueError, SyntaxError):
            continue
        data, weight, strides = parts
        if len(data) != 5 or len(weight) != 7 or len(strides) != 2 or data[4] != 16 or weight[4:] != (4, 16, 4):
            continue
        key = (data[0], data[1] * 16, data[2], data[3], weight[0] * 16, weight[2], weight[3], strides[0], strides[1])
        seen[key] = seen.get(key, 0) + 1
    names = ('n', 'c_in', 'h', 'w', 'c_out', 'kh', 'kw', 'stride_h', 'stride_w')
    return [dict(zip(names, k), count=v) for k, v in sorted(seen.items())]


def load_corpus() -> List[dict]:
    with open(CORPUS_PATH) as f:
        return json.load(f)['shapes']


def set_table(entries: List[dict]) -> None:
    """Hand a list of entries (dicts with the fields of ``unit_tile_entry``; missing ones 0) to the library."""
    global _VERSION
    L = _lib.lib()
    arr = (_lib.TileEntry * max(1, len(entries)))()
    for i, e in enumerate(entries):
        for f in FIELDS:
            setattr(arr[i], f, int(e.get(f, 16 if f == 'c_block' else 0)))
    _lib.check(L.unit_tile_table_set(arr, len(entries)), 'unit_tile_table_set')
    _VERSION += 1


def load_default_table() -> int:
    """Loads ``tile_table.json`` if it exists; returns the number of entries."""
    if not os.path.exists(TABLE_PATH):
        return 0
    with open(TABLE_PATH) as f:
        entries = json.load(f).get('entries', [])
    set_table(entries)
    return len(entries)


def main(argv: List[str]) -> int:
    if len(argv) == 3 and argv[1] == 'corpus':
        with open(argv[2]) as f:
            shapes = parse_shape_log(f)
        with open(CORPUS_PATH, 'w') as f:
            json.dump({'source': "were/UNIT cpu-shapes.log: unique int8 NCHW16c convolution shapes (pre-padded sizes), with the "
                                 "number of rows that carry each",
                       'shapes': shapes}, f, indent=0)
        print(f'{len(shapes)} shapes -> {CORPUS_PATH}')
        return 0
    print('usage: python -m unit_b200.tile_table corpus <cpu-shapes.log>')
    return 2


if __name__ == '__main__':
    sys.exit(main(sys.argv))
