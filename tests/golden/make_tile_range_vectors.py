"""Writes tests/golden/tile_ranges.json: the two known-answer cases for the tile-range stage.

The cases are the ones the reference's own unit tests assert (tests/rasterizer_test.cpp:66-110 there):
ten keys built as (tile << 32) | depth for a 40x30 image (3x2 tiles -> 7 range entries).  They are
restated here as data (tile ids, depth values, expected ranges); this script only packs them into keys.
Run: python tests/golden/make_tile_range_vectors.py
"""
import json
import os

CASES = [
    dict(name="every_tile_present", image_height=30, image_width=40,
         tiles=[0, 1, 1, 2, 3, 3, 4, 5, 5, 5], depths=[40, 20, 50, 60, 10, 20, 20, 40, 30, 50],
         expected=[0, 1, 3, 4, 6, 7, 10]),
    dict(name="tiles_without_entries", image_height=30, image_width=40,
         tiles=[0, 1, 1, 3, 3, 3, 3, 5, 5, 5], depths=[40, 20, 50, 60, 10, 20, 20, 40, 30, 50],
         expected=[0, 1, 3, 3, 7, 7, 10]),
]

for c in CASES:
    c["keys"] = [(t << 32) | d for t, d in zip(c["tiles"], c["depths"])]

out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "tile_ranges.json")
with open(out, "w") as f:
    json.dump(CASES, f, indent=1)
print("wrote", out)
