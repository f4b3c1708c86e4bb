"""Routing traces: the text the reference's runner appends when NVMAI_ROUTE_TRACE names a
file (`recordRouteTrace`, RealForwardRunner.swift:1208-1237), one line per decode layer and
token, `position layer e0 e1 ... e7`, read back as a routing source for replay.

A replay hands the recorded expert ids to `MoE.routed_partial` (the routed kernels run from
given ids), so a benchmark sees the popularity and the token-to-token reuse of a real run
instead of uniform or Zipf draws.  `synthesize` writes a trace with a chosen reuse rate in
the same format for machines that hold no recorded trace.
"""
from __future__ import annotations

import io
import os
from dataclasses import dataclass

import numpy as np


class RouteTraceError(ValueError):
    """A malformed trace line; the message carries the 1-based line number."""


@dataclass
class RouteTrace:
    positions: np.ndarray      # int64 [n]
    layers: np.ndarray         # int32 [n]
    experts: np.ndarray        # int32 [n, top_k], in the router's rank order
    num_experts: int

    @property
    def top_k(self) -> int:
        return int(self.experts.shape[1])

    def __len__(self) -> int:
        return int(self.positions.shape[0])

    def layer_ids(self) -> list[int]:
        return sorted(int(v) for v in np.unique(self.layers))

    def layer_rows(self, layer: int) -> tuple[np.ndarray, np.ndarray]:
        """-> (positions ascending, expert ids [rows, top_k]) of one layer; a position that was recorded twice
        (a re-run of the same token) keeps its last record."""
        sel = np.nonzero(self.layers == layer)[0]
        pos = self.positions[sel]
        order = np.argsort(pos, kind="stable")
        pos, ids = pos[order], self.experts[sel][order]
        if pos.size > 1:
            last = np.append(pos[1:] != pos[:-1], True)
            pos, ids = pos[last], ids[last]
        return pos, ids

    def batch(self, layer: int, first_row: int, rows: int) -> np.ndarray:
        """`rows` consecutive recorded tokens of a layer starting at row `first_row`, wrapping round."""
        _, ids = self.layer_rows(layer)
        if ids.shape[0] == 0:
            raise RouteTraceError(f"layer {layer} has no record")
        take = (first_row + np.arange(rows)) % ids.shape[0]
        return np.ascontiguousarray(ids[take])

    def stats(self, window: int = 128) -> dict:
        """Mean over layers of: the share of a token's experts that the previous token of the same layer also chose
        (`reuse`), the distinct experts per `window` consecutive tokens, and the distinct experts overall."""
        reuse, distinct_w, distinct_all = [], [], []
        for layer in self.layer_ids():
            _, ids = self.layer_rows(layer)
            n = ids.shape[0]
            if n > 1:
                same = [(np.isin(ids[t], ids[t - 1])).mean() for t in range(1, n)]
                reuse.append(float(np.mean(same)))
            for s in range(0, max(n - window + 1, 1), window):
                distinct_w.append(np.unique(ids[s:s + window]).size)
            distinct_all.append(np.unique(ids).size)
        return {"records": len(self), "layers": len(self.layer_ids()),
                "reuse": float(np.mean(reuse)) if reuse else 0.0,
                "distinct_per_window": float(np.mean(distinct_w)) if distinct_w else 0.0, "window": window,
                "distinct_per_layer": float(np.mean(distinct_all)) if distinct_all else 0.0}

    def format(self) -> str:
        out = io.StringIO()
        for p, l, row in zip(self.positions, self.layers, self.experts):
            out.write(f"{int(p)} {int(l)} " + " ".join(str(int(e)) for e in row) + "\n")
        return out.getvalue()


def from_route_log(log, first_position: int = 0, *, num_experts: int = 256) -> RouteTrace:
    """The routing a decode step recorded on the device (`MoE.read_route_log`: [layers][top_k], or
    `read_route_log_rows`: [layers][rows][top_k]) as trace records: row r of the step is position
    first_position + r, layers in order.  `.format()` then gives the reference's NVMAI_ROUTE_TRACE lines
    (`position layer e0..e7`, RealForwardRunner.swift:1208-1237)."""
    log = np.asarray(log)
    if log.ndim == 2:
        log = log[:, None, :]
    layers, rows, k = log.shape
    pos = np.repeat(np.arange(rows, dtype=np.int64) + first_position, layers)
    lay = np.tile(np.arange(layers, dtype=np.int32), rows)
    exp = log.transpose(1, 0, 2).reshape(rows * layers, k).astype(np.int32)
    return RouteTrace(positions=pos, layers=lay, experts=exp, num_experts=num_experts)


def parse(source, *, num_experts: int = 256, top_k: int = 8, num_layers: int | None = None) -> RouteTrace:
    """`source`: a path, or the text itself.  Every line must read `position layer e0 .. e{top_k-1}` with
    0 <= e < num_experts, no expert twice in a line and (when given) layer < num_layers; blank lines are skipped.
    A trailing line without its newline (a run that was cut off while writing) is dropped if it is short."""
    if isinstance(source, (str, os.PathLike)) and "\n" not in str(source) and os.path.exists(source):
        with open(source, "r", encoding="utf-8") as fh:
            text = fh.read()
    else:
        text = str(source)
    lines = text.split("\n")
    cut_off = not text.endswith("\n")
    pos, lay, ids = [], [], []
    for n, line in enumerate(lines, 1):
        fields = line.split()
        if not fields:
            continue
        if len(fields) != 2 + top_k:
            if cut_off and n == len(lines) and len(fields) < 2 + top_k:
                continue
            raise RouteTraceError(f"line {n}: {len(fields)} fields, expected {2 + top_k}")
        try:
            vals = [int(f) for f in fields]
        except ValueError:
            raise RouteTraceError(f"line {n}: not an integer") from None
        p, l, row = vals[0], vals[1], vals[2:]
        if p < 0 or l < 0 or (num_layers is not None and l >= num_layers):
            raise RouteTraceError(f"line {n}: position {p} / layer {l} out of range")
        if min(row) < 0 or max(row) >= num_experts:
            raise RouteTraceError(f"line {n}: expert id outside 0..{num_experts - 1}")
        if len(set(row)) != top_k:
            raise RouteTraceError(f"line {n}: an expert appears twice")
        pos.append(p); lay.append(l); ids.append(row)
    return RouteTrace(np.asarray(pos, dtype=np.int64), np.asarray(lay, dtype=np.int32),
                      np.asarray(ids, dtype=np.int32).reshape(len(ids), top_k), num_experts)


def synthesize(positions: int, layers: int, *, num_experts: int = 256, top_k: int = 8, reuse: float = 0.38,
               zipf: float = 0.6, seed: int = 1) -> RouteTrace:
    """A trace in the recorded format: each token keeps each of its predecessor's experts with probability `reuse`
    and draws the others from a Zipf(`zipf`) popularity over a per-layer permutation of the experts (0.38 is the
    consecutive-token reuse the reference's notes report for its model)."""
    rng = np.random.default_rng(seed)
    p = np.arange(1, num_experts + 1, dtype=np.float64) ** -zipf
    p /= p.sum()
    pos, lay, ids = [], [], []
    prev = {}
    perms = [rng.permutation(num_experts) for _ in range(layers)]
    for t in range(positions):
        for l in range(layers):
            keep = [e for e in prev.get(l, []) if rng.random() < reuse]
            row = list(keep)
            while len(row) < top_k:
                e = int(perms[l][rng.choice(num_experts, p=p)])
                if e not in row:
                    row.append(e)
            rng.shuffle(row)
            prev[l] = row
            pos.append(t); lay.append(l); ids.append(row)
    return RouteTrace(np.asarray(pos, dtype=np.int64), np.asarray(lay, dtype=np.int32),
                      np.asarray(ids, dtype=np.int32), num_experts)
