"""Reader of the profiled database the search runs against (CSV files written by the profilers).

File formats (unchanged from the reference, profiler/op_profiler.py:461-487, profiler/comm_profiler.py:160-169,
profiler/p2p_band_profiler.py:58-62):
  {model}_{size}_mbs{m}_tp{t}_algo{a}.csv : op_name, forward-compute, backward-compute (us), input_size,
        output_size, weights, activations, fwd_reserved, bwd_reserved (MB)
        optional extra columns (this framework): fwd_overlap_comm, bwd_overlap_comm (us) = the part of the op's
        own collective that the fused kernels hide under the math
  prim_{model}_{size}_{collective}_{n}gpus.csv : data_size(MB), time(ms)
  p2p_intra_node.csv / p2p_inter_node.csv   : row 0 sizes (MB, powers of two), row 1 bandwidth (GB/s ~ MB/ms)
"""
from __future__ import annotations

import csv
import math
from typing import Dict, List, Optional, Sequence

MISSING = 1000000  # value of a table cell that no file filled in


class ProfileDB:
    FIELDS = ("fwd", "bwd", "in_mb", "out_mb", "weights", "acts", "res_fwd", "res_bwd", "fwd_ovl", "bwd_ovl")

    def __init__(self, model_name: str, model_size: str, path: str, mbs_list: Sequence[int], max_tp: int,
                 unique_ops: Sequence[str], use_reserved: bool = True, verbose: bool = True):
        self.model_name, self.model_size, self.path = model_name, model_size, path
        self.mbs_list = list(mbs_list)
        self.mbs_index = {m: i for i, m in enumerate(self.mbs_list)}
        small = (model_name == "gpt" and model_size == "350M") or (model_name == "t5" and model_size == "220M")
        top = min(max_tp, 4 if small else 8)
        self.tp_list = []
        t = 1
        while t <= top:
            self.tp_list.append(t)
            t *= 2
        self.algos = [0] if model_name == "t5" else [0, 1]
        size = "11B" if (model_name == "t5" and model_size == "22B") else model_size
        # table[field][op][mbs_idx][log2 tp][algo]
        self.table: Dict[str, Dict[str, list]] = {f: {} for f in self.FIELDS}
        for f in self.FIELDS:
            fill = 0.0 if f in ("fwd_ovl", "bwd_ovl") else MISSING
            for op in unique_ops:
                self.table[f][op] = [[[fill for _ in self.algos] for _ in self.tp_list] for _ in self.mbs_list]
        self.has_overlap_columns = False
        for mbs in self.mbs_list:
            for tp in self.tp_list:
                for algo in self.algos:
                    stem = f"gpt_scale-layer" if model_name == "scale-layer" else f"{model_name}_{size}"
                    fname = f"{path}{stem}_mbs{mbs}_tp{tp}_algo{algo}.csv"
                    try:
                        with open(fname) as fh:
                            rows = list(csv.reader(fh))
                        mi, ti = self.mbs_index[mbs], int(math.log(tp, 2))
                        for row in rows[1:]:
                            op = row[0]
                            cells = (("fwd", 1), ("bwd", 2), ("in_mb", 3), ("out_mb", 4), ("weights", 5), ("acts", 6))
                            for f, c in cells:
                                self.table[f][op][mi][ti][algo] = float(row[c])
                            if use_reserved:
                                self.table["res_fwd"][op][mi][ti][algo] = float(row[7])
                                self.table["res_bwd"][op][mi][ti][algo] = float(row[8])
                            if len(row) > 10:
                                self.has_overlap_columns = True
                                self.table["fwd_ovl"][op][mi][ti][algo] = float(row[9])
                                self.table["bwd_ovl"][op][mi][ti][algo] = float(row[10])
                    except Exception:  # noqa: BLE001 - a missing table leaves the sentinel, like the reference
                        if verbose:
                            print(f"file ({fname}) not exist, or the file is not formatted as expected.")
        # collectives
        prims = {"gpt": ["all_gather", "all_reduce", "reduce_scatter", "all_to_all"],
                 "scale-layer": ["all_gather", "all_reduce", "reduce_scatter", "all_to_all"],
                 "bert": ["all_gather", "all_reduce", "reduce_scatter", "all_to_all"],
                 "vit": ["all_gather", "all_reduce", "reduce_scatter", "all_to_all"],
                 "t5": [], "resnet": ["all_gather", "all_to_all"]}[model_name]
        self.collective: Dict[str, Dict[int, Dict[str, float]]] = {}
        for prim in prims:
            self.collective[prim] = {}
            for n in self.tp_list[1:]:
                stem = "gpt_scale-layer" if model_name == "scale-layer" else f"{model_name}_{size}"
                tab: Dict[str, float] = {}
                with open(f"{path}prim_{stem}_{prim}_{n}gpus.csv") as fh:
                    for row in list(csv.reader(fh))[1:]:
                        tab[row[0]] = float(row[1])
                self.collective[prim][n] = tab
        # p2p bandwidth
        self.intra_band = self._band(path + "p2p_intra_node.csv")
        inter = self._band(path + "p2p_inter_node.csv")
        if self.intra_band is None and verbose:
            print("intra-node bandwidth file is not found.")
        if inter is None:
            if verbose:
                print("inter-node bandwidth file is not found, using intra-node bandwidth instead.")
            inter = self.intra_band
        self.inter_band = inter

    @staticmethod
    def _band(fname: str) -> Optional[List[float]]:
        try:
            with open(fname) as fh:
                rows = list(csv.reader(fh))
            return [float(x) for x in rows[1]]
        except Exception:  # noqa: BLE001
            return None

    def get(self, field: str, op: str, mbs: int, tp: int, algo: int) -> float:
        return self.table[field][op][self.mbs_index[mbs]][int(math.log(tp, 2))][algo]

    def collective_time(self, prim: str, n: int, size_mb: float) -> float:
        """Exact-size lookup (ms); 100000 when the size was never profiled."""
        assert n > 1
        if prim in ("all_reduce", "all_gather", "reduce_scatter", "all_to_all"):
            tab = self.collective[prim][n]
            key = "{:.0f}".format(float(size_mb))
            if key in tab:
                return tab[key]
            key = "{:.0f}".format(float(size_mb) - 1)
            if key in tab:
                return tab[key]
            return 100000
        if prim == "split":
            return 0
        return 100000

    @staticmethod
    def _bucket(band: List[float], size_mb: float) -> float:
        if size_mb > 0:
            idx = int(math.log(size_mb, 2))
            if idx >= 1:
                idx -= 1
            return (band[-1] if idx >= len(band) else band[idx]) * 0.001
        return 1

    def intra_bandwidth(self, size_mb: float) -> float:
        return self._bucket(self.intra_band, size_mb)

    def inter_bandwidth(self, size_mb: float) -> float:
        return self._bucket(self.inter_band, size_mb)
