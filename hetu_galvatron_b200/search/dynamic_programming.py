"""Dynamic-programming driver of the strategy search.

``DPAlg`` solves one pipeline stage: choose a strategy per layer minimising time under a memory budget
(knapsack over MB), through the C++ core (csrc/dp_core.cpp) or a NumPy fallback with the same results.
``DpOnModel`` builds the per-layer memory / time tables and the inter-layer resharding costs for one pipeline
degree, runs ``DPAlg`` per stage and picks the vocab-tp degree with the pipeline cost model.
Reference behaviour: galvatron/core/search_engine/dynamic_programming.py:7-126 (DPAlg), :128-565 (DpOnModel).
"""
from __future__ import annotations

import hashlib
import threading

import numpy as np

from .cost_model import OtherTimeCostModel, pipeline_costmodel

_CORE = None


def _core():
    global _CORE
    if _CORE is None:
        from .. import _build
        _CORE = _build.load_pybind("dp_core")
    return _CORE


_FIT_CACHE: dict = {}                 # digest of a stage problem -> its solution
_MARK_POOL = threading.local()        # one buffer per thread: --parallel_search runs fits on a thread pool


def _mark_scratch(layers: int, mem: int, strategies: int) -> np.ndarray:
    """Back-pointer table for one fit. A search runs thousands of fits of similar size, each of which overwrites the whole
    table and reads it back before returning, so they share one buffer (tens to hundreds of MB) instead of allocating and
    page-faulting a new one per fit."""
    need = layers * mem * strategies
    buf = getattr(_MARK_POOL, "buf", None)
    if buf is None or buf.size < need:
        buf = _MARK_POOL.buf = np.empty(need, dtype=np.int32)
    return buf[:need].reshape(layers, mem, strategies)


class DPAlg:
    def __init__(self, max_mem=8200, other_mem_cost=None, other_time_cost=None, layer_num=24, strategy_num=4,
                 strategy_set=None, fine_grained_mode=True, use_cpp_core=True) -> None:
        assert other_mem_cost is not None
        self.max_mem = max_mem + 1
        self.layer_num, self.strategy_num = layer_num, strategy_num
        self.other_mem_cost, self.other_time_cost = other_mem_cost, other_time_cost
        self._f = np.zeros((self.max_mem, strategy_num), dtype=np.float64)
        self._mark = None            # back-pointers [layer, memory, strategy]: taken from the scratch pool when a fit needs them
        self.v_data = self.inter_cost = self.intra_cost = None
        self.use_cpp_core, self.strategy_set, self.fine_grained_mode = use_cpp_core, strategy_set, fine_grained_mode

    def set_v_and_cost(self, v: np.ndarray, intra_layer_cost: np.ndarray, inter_layer_cost: np.ndarray):
        L, S = self.layer_num, self.strategy_num
        assert v.shape == (L, S) and intra_layer_cost.shape == (L, S) and inter_layer_cost.shape == (L, S, S)
        self.v_data = np.ascontiguousarray(v, dtype=np.int32)
        self.inter_cost = np.ascontiguousarray(inter_layer_cost, dtype=np.float64)
        self.intra_cost = np.ascontiguousarray(intra_layer_cost, dtype=np.float64)

    def _fit_uniform(self):
        """Coarse mode: one strategy for the whole stage, per vocab-tp key the cheapest that fits."""
        keys = list(self.other_mem_cost)
        res = {k: np.full(self.layer_num, -1, dtype=np.int32) for k in keys}
        cost = {k: np.inf for k in keys}
        remain = {k: -1 for k in keys}
        for k in keys:
            for i in range(self.strategy_num):
                if self.strategy_set[i][1] != k:
                    continue
                t = sum(self.intra_cost[:, i]) + sum(self.inter_cost[:, i, i]) + self.other_time_cost[k]
                m = sum(self.v_data[:, i]) + self.other_mem_cost[k]
                if self.max_mem - 1 - m >= 0 and cost[k] > t:
                    remain[k], cost[k] = self.max_mem - 1 - m, t
                    res[k] = np.full(self.layer_num, i, dtype=np.int32)
        return cost, res, remain

    def _fit_numpy(self):
        """Same recurrence as the C++ core, vectorised over (memory, previous strategy)."""
        L, V, S = self.layer_num, self.max_mem, self.strategy_num
        self._mark = _mark_scratch(L, V, S)
        f = self._f.copy()
        for i in range(L):
            new = np.full((V, S), np.inf)
            for s in range(S):
                m = int(self.v_data[i, s])
                if m >= V:
                    self._mark[i, :, s] = -1
                    continue
                cand = (f[: V - m, :] + self.inter_cost[i, :, s][None, :]) + self.intra_cost[i, s]
                best = np.argmin(cand, axis=1)
                self._mark[i, m:, s] = best
                new[m:, s] = cand[np.arange(V - m), best]
                self._mark[i, :m, s] = -1
            f = new
        self._f[:] = f
        total, remain = {}, {}
        res = {k: np.full(L, -1, dtype=np.int32) for k in self.other_mem_cost}
        for k, other in self.other_mem_cost.items():
            v = V - 1 - other
            if v < 0 or not (f[v].min() < np.inf):
                total[k], remain[k] = np.inf, -1
                continue
            idx = int(np.argmin(f[v]))
            total[k] = f[v, idx] + self.other_time_cost[k]
            res[k][L - 1] = idx
            for i in range(L - 1, 0, -1):
                cur = idx
                idx = int(self._mark[i, v, cur])
                v -= int(self.v_data[i, cur])
                res[k][i - 1] = idx
            remain[k] = int(v - self.v_data[0, idx])
        return total, res, remain

    def fit(self):
        if not self.fine_grained_mode:
            return self._fit_uniform()
        # The outer loops of a search (micro-batch counts, vocab degrees, sequence-parallel variants, pipeline stages) pose
        # the same stage problem again and again: about two thirds of the fits of a Llama-7B search repeat an earlier one.
        h = hashlib.sha1()
        for a in (self.v_data, self.intra_cost, self.inter_cost):
            h.update(a.tobytes())
        h.update(repr((self.v_data.shape, self.max_mem, self.use_cpp_core, sorted((int(k), int(v)) for k, v in self.other_mem_cost.items()),
                       sorted((int(k), float(v)) for k, v in self.other_time_cost.items()))).encode())
        key = h.digest()
        hit = _FIT_CACHE.get(key)
        if hit is None:
            hit = self._fit_capped()
            if len(_FIT_CACHE) >= 16384:
                _FIT_CACHE.clear()
            _FIT_CACHE[key] = hit
        total, res, remain = hit
        return dict(total), {k: list(v) for k, v in res.items()}, dict(remain)

    def _fit_capped(self):
        # Above the sum over layers of the largest memory cost that fits at all, the budget binds nowhere: every table
        # row there repeats the row at that sum, with the same back-pointers. Solving up to that row and starting the
        # back-tracking of every vocab key at min(its row, that row) gives the same costs and plans in a smaller table.
        V = self.max_mem
        fits = np.where(self.v_data < V, self.v_data, 0)
        cap = int(fits.max(axis=1).astype(np.int64).sum()) + 1
        if cap < V:
            shift = V - cap
            full_other, full_f = self.other_mem_cost, self._f
            self.max_mem, self._f = cap, np.ascontiguousarray(full_f[:cap])
            self.other_mem_cost = {k: max(int(m) - shift, 0) for k, m in full_other.items()}
            try:
                total, res, remain = self._fit_table()
            finally:
                self.max_mem, self._f, self.other_mem_cost = V, full_f, full_other
            for k, m in full_other.items():
                if remain[k] >= 0:
                    remain[k] += max(0, (V - 1 - int(m)) - (cap - 1))
            return total, res, remain
        return self._fit_table()

    def _fit_table(self):
        if self.use_cpp_core:
            res = {k: np.full(self.layer_num, -1, dtype=np.int32) for k in self.other_mem_cost}
            other_mem = {int(k): int(v) for k, v in self.other_mem_cost.items()}
            other_time = {int(k): float(v) for k, v in self.other_time_cost.items()}
            self._mark = _mark_scratch(self.layer_num, self.max_mem, self.strategy_num)      # the core writes every cell
            total, remain = _core().dynamic_programming_core(self.layer_num, self.max_mem, self.strategy_num, self.v_data,
                                                             self._mark, self._f, self.inter_cost, self.intra_cost,
                                                             other_mem, other_time, res)
            return total, {k: list(v) for k, v in res.items()}, remain
        total, res, remain = self._fit_numpy()
        return total, {k: list(v) for k, v in res.items()}, remain


def _same_except(s1, s2, ignore=()) -> bool:
    """Strategies equal in (pp, tp, dp) and in every flag not listed in ``ignore``."""
    if list(s1[:3]) != list(s2[:3]):
        return False
    a, b = s1[-1], s2[-1]
    keys = (set(a) | set(b)) - set(ignore)
    return all(k in a and k in b and a[k] == b[k] for k in keys)


class DpOnModel:
    def __init__(self, strategies_set, memcost_model, timecost_model, model_args_list=None, train_args_list=None,
                 parallel_args_list=None, profile_model_args_list=None, profile_hardware_args_list=None, max_mem=8192,
                 layer_num=24, sequence_len=[512], multi_layer_type=False, pp_stage_dict=None, search_history=None,
                 comm_coe_dict={}, gpu_num=8, mem_cache=True, model_microbatch_after_dp=False, pipeline_type="gpipe",
                 config=None, logger=None):
        self.strategies_set = strategies_set
        self.memcost_model, self.timecost_model = memcost_model, timecost_model
        self.model_args_list, self.train_args_list, self.parallel_args_list = model_args_list, train_args_list, parallel_args_list
        self.profile_model_args_list, self.profile_hardware_args_list = profile_model_args_list, profile_hardware_args_list
        self.max_mem, self.layer_num, self.sequence_len = max_mem, layer_num, sequence_len
        self.n_gpu = strategies_set[0][0] * strategies_set[0][1] * strategies_set[0][2]
        self.ppdeg_set = np.unique(np.array([s[0] for s in strategies_set], dtype=np.int32))
        self.multi_layer_type, self.search_history = multi_layer_type, search_history
        self.comm_coe_dict, self.gpu_num, self.config, self.logger = comm_coe_dict, gpu_num, config, logger
        if multi_layer_type:
            assert isinstance(layer_num, list)
            self.total_layer_num = sum(layer_num)
            for lst in (model_args_list, train_args_list, parallel_args_list, profile_model_args_list, profile_hardware_args_list):
                assert isinstance(lst, list) and len(lst) == len(layer_num)
            assert isinstance(pp_stage_dict, dict)
            for pp in self.ppdeg_set:
                if pp > 1:
                    assert pp in pp_stage_dict and sum(pp_stage_dict[pp]) == self.total_layer_num
            self.pp_stage_dict = pp_stage_dict
            self.pp_stage_dict.setdefault(1, [self.total_layer_num])
        # keep 20 % of a large budget free for the caching allocator
        self.mem_cache = 0
        if max_mem // 1024 > 20 and mem_cache:
            self.mem_cache = int(max_mem * 0.2)
            self.max_mem -= self.mem_cache
        self.model_microbatch_after_dp, self.pipeline_type = model_microbatch_after_dp, pipeline_type
        # Memory resolution of the knapsack. The reference works in MB, which for a 180 GB device makes tables of
        # > 140 k rows per layer; beyond 32 Ki rows the unit is coarsened (costs rounded up, so plans stay feasible).
        unit = getattr(config, "memory_granularity_mb", 0) or 0
        self.mem_unit = int(unit) if unit > 0 else max(1, -(-int(self.max_mem) // 32768))

    def match_strategy(self, s1, s2, except_keys=[]):
        return _same_except(s1, s2, except_keys)

    # ------------------------------------------------------------------ tables
    def _kw(self, i):
        return dict(model_args=self.model_args_list[i], train_args=self.train_args_list[i],
                    parallel_args=self.parallel_args_list[i], profile_model_args=self.profile_model_args_list[i])

    def _intra_costs(self, strategy_set, bsz, chunks):
        rows = []
        for i, n in enumerate(self.layer_num):
            b = bsz / chunks[i] if self.model_microbatch_after_dp else bsz
            # costs of one micro-batch carry their share of the once-per-step optimizer time
            share = 1.0 / chunks[i] if self.model_microbatch_after_dp else 1.0
            row = []
            for s in strategy_set:
                kw = dict(profile_hardware_args=self.profile_hardware_args_list[i], logger=self.logger, **self._kw(i))
                try:
                    m = self.timecost_model(s, b, with_optimizer=False, **kw)
                    coe = 0.001 * getattr(self.profile_hardware_args_list[i], "costmodel_coe", 1.0)
                    row.append(m.gen_result() + m.optimizer_ms() * coe * share)
                except TypeError:         # a cost-model class without the optimizer term
                    row.append(self.timecost_model(s, b, **kw).gen_result())
            rows.append(np.array(row, dtype=np.float64).reshape(1, -1).repeat(n, axis=0))
        return np.concatenate(rows, axis=0)

    def _memory_tables(self, strategy_set, pp_deg, bsz, mbsz, min_tp, max_tp, vsp, embed_sdp):
        """Per-stage [layers, strategies] MB tables (one table shared by all stages for GPipe) + other memory."""
        other_mem = {}
        stages = [0] if self.pipeline_type == "gpipe" else list(range(pp_deg))
        tables = []
        for stage_idx in stages:
            blocks = []
            for i, n in enumerate(self.layer_num):
                extra = {} if self.pipeline_type == "gpipe" else {"stage_idx": stage_idx}
                costs = [self.memcost_model(s, bsz, mbsz=mbsz, min_tp=min_tp, max_tp=max_tp, vsp=vsp, embed_sdp=embed_sdp,
                                            logger=self.logger, **extra, **self._kw(i)).get_memory_cost() for s in strategy_set]
                if stage_idx == 0 and i == 0:
                    for k, v in costs[0]["other"].items():
                        other_mem[k] = np.ceil(v).astype(int)
                v = np.ceil(np.array([c["enc_total"] for c in costs])).astype(np.int32)
                blocks.append(v.reshape(1, -1).repeat(n, axis=0))
            tables.append(np.concatenate(blocks, axis=0))
        if self.pipeline_type == "gpipe":
            tables = tables * pp_deg
        return tables, other_mem

    def _inter_costs(self, strategy_set, mbsz, min_tp):
        """Resharding cost between adjacent layers (+ tiny biases that order otherwise equal choices:
        plain < sp (1e-10) < zero3 (1e-9) < checkpoint (2e-9) < zero3+checkpoint (3e-9))."""
        S = len(strategy_set)
        elem = 4 if self.config.mixed_precision == "fp32" else 2
        mats = []
        for idx, n in enumerate(self.layer_num):
            sample = self.sequence_len[idx] * self.config.hidden_size * elem
            m = np.zeros((S, S))
            for i, si in enumerate(strategy_set):
                for j, sj in enumerate(strategy_set):
                    grows = sj[1] > si[1]
                    flips = shrink_flip = False
                    if "tp" in sj[-1] and "tp" in si[-1]:
                        differ = sj[-1]["tp"] != si[-1]["tp"]
                        flips = sj[1] == si[1] and differ
                        shrink_flip = si[1] * si[2] == 8 and si[1] == 4 and sj[1] == 2 and differ
                    sp_change = self.config.sequence_parallel and sj[1] != si[1]
                    if grows or flips or shrink_flip or sp_change:
                        wide = max(sj[1], si[1])
                        m[i, j] = (wide - 1) / wide * mbsz * (wide // min_tp) * sample
                    tp_size, dp_size = max(sj[1], si[1]), min(sj[2], si[2])
                    if tp_size == 1 or dp_size == 1:
                        key = "%d" % tp_size
                        coe = self.comm_coe_dict[key] if key in self.comm_coe_dict else self.comm_coe_dict["%d_1" % tp_size]
                    else:
                        info = sj[-1] if sj[1] > si[1] else si[-1]
                        assert "tp" in info and info["tp"] in (0, 1)
                        coe = self.comm_coe_dict["%d_%d" % (tp_size, 1 if info["tp"] else 0)]
                    m[i, j] = m[i, j] * coe * 1e-7
                    if i == j:
                        continue
                    if _same_except(si, sj, ["sp"]) and sj[-1].get("sp"):
                        m[i, j] = 1e-10
                    if _same_except(si, sj, ["fsdp"]) and sj[-1].get("fsdp"):
                        m[i, j] = 1e-9
                    if _same_except(si, sj, ["cpt"]) and sj[-1].get("cpt"):
                        m[i, j] = 2e-9
                    if _same_except(si, sj, ["fsdp", "cpt"]):
                        if sj[-1].get("fsdp") and sj[-1].get("cpt"):
                            m[i, j] = 3e-9
                        if (not _same_except(si, sj, ["fsdp"]) and not _same_except(si, sj, ["cpt"])
                                and si[-1].get("fsdp") and sj[-1].get("cpt")):
                            m[i, j] = 1e-9
            mats.append(np.expand_dims(m, 0).repeat(n, axis=0))
        inter = np.concatenate(mats, axis=0)
        inter[0, :, :] = 0
        return inter

    # ------------------------------------------------------------------ one pipeline degree
    def _build_dp_and_run_multi_layer_type(self, pp_deg, bsz, mbsz, min_tp, max_tp, vsp, embed_sdp, sp_search):
        cfg = self.config
        chunks = None
        if self.model_microbatch_after_dp:
            dp_size = self.gpu_num // pp_deg
            chunks = [pa.optimal_chunk_func(bsz * min_tp // dp_size, [pp_deg, min_tp, dp_size], mbsz, min_tp)
                      for pa in self.parallel_args_list]
        strategy_set = [s for s in self.strategies_set if s[0] == pp_deg]
        S = len(strategy_set)
        intra = self._intra_costs(strategy_set, bsz, chunks)
        cheapest = np.argmin(intra, axis=1)
        other_time = OtherTimeCostModel(mbsz, pp_deg, self.n_gpu, vsp, embed_sdp, min_tp, max_tp, self.sequence_len,
                                        model_args=self.model_args_list[0], train_args=self.train_args_list[0],
                                        parallel_args=self.parallel_args_list[0],
                                        profile_model_args=self.profile_model_args_list[0],
                                        profile_hardware_args=self.profile_hardware_args_list[0], logger=self.logger).gen_result()
        v_tables, other_mem = self._memory_tables(strategy_set, pp_deg, bsz, mbsz, min_tp, max_tp, vsp, embed_sdp)
        inter = self._inter_costs(strategy_set, mbsz, min_tp)
        stage_layers = self.pp_stage_dict[pp_deg]
        fine = cfg.fine_grained_mode != 0

        def gather_buffer_mb(coarse: bool) -> float:
            use = cfg.sequence_parallel and (coarse or (getattr(cfg, "global_memory_buffer", True) and sp_search != 2))
            if not use:
                return 0
            mb = mbsz / min_tp * max_tp * cfg.hidden_size * max(self.sequence_len) * 4 / 1024 / 1024
            return mb / 2 if cfg.mixed_precision else mb

        def solve(columns, local_set):
            """DP over every stage restricted to strategy columns ``columns``."""
            costs, plans, remains, mems = [], [], [], []
            flags = {k: [False] * pp_deg for k in other_mem}
            start = 0
            for st in range(pp_deg):
                n = stage_layers[st]
                extra = int(gather_buffer_mb(coarse=not fine))
                U = self.mem_unit
                o_mem = {k: -(-int(v[st] + extra) // U) for k, v in other_mem.items()}
                o_time = {k: v[st] for k, v in other_time[0].items()}
                dp = DPAlg(self.max_mem // U, o_mem, o_time, n, len(columns), local_set, cfg.fine_grained_mode)
                rows = slice(start, start + n)
                v_units = v_tables[st][rows][:, columns] if U == 1 else -(-v_tables[st][rows][:, columns] // U)
                dp.set_v_and_cost(v_units.astype(np.int32), intra[rows][:, columns], inter[rows][:, columns][:, :, columns])
                cost, res, remain = dp.fit()
                remain = {k: (r * U if r >= 0 else r) for k, r in remain.items()}      # back to MB
                mem = {k: 0 for k in o_mem}
                for k in cost:
                    if remain[k] == -1:
                        res[k] = None
                    flags[k][st] = res[k] is not None and (np.array(res[k]) == cheapest[rows]).all()
                    if res[k] is not None:
                        res[k] = [local_set[x] for x in res[k]]
                    mem[k] = self.max_mem // U * U - remain[k] if remain[k] >= 0 else np.inf
                costs.append(cost); plans.append(res); remains.append(remain); mems.append(mem)
                start += n
            return costs, plans, remains, mems, flags

        def pick_vtp(costs, plans, best_cost):
            """Vocab-tp key with the lowest pipeline cost (when the pipeline cost model is on)."""
            vtp = -1
            for k in other_time[0]:
                if any(k not in p for p in plans):
                    continue            # no memory profile for this vocab-tp degree
                per_stage = [p[k] for p in plans]
                if self.model_microbatch_after_dp:
                    if None in per_stage:
                        continue
                    flat = [s for stage in per_stage for s in stage]
                    c = pipeline_costmodel(self.timecost_model, self.layer_num, self.model_args_list, self.train_args_list,
                                           self.parallel_args_list, self.profile_model_args_list,
                                           self.profile_hardware_args_list, flat, stage_layers, chunks, bsz, min_tp,
                                           other_time[1][k], self.logger)
                    if best_cost > c:
                        best_cost, vtp = c, k
                else:
                    best_cost = sum(c[k] for c in costs)
            return best_cost, vtp

        if not fine:
            best, vtp = np.inf, -1
            final = ([], [], [])
            flags = {k: [False] * pp_deg for k in other_mem}
            remains = mems = []
            for si in range(S):
                costs, plans, remains, mems, flags = solve([si], [strategy_set[si]])
                new_best, k = pick_vtp(costs, plans, best)
                if k != -1:
                    best, vtp = new_best, k
                    final = ([p[k] for p in plans], [r[k] for r in remains], [m[k] for m in mems])
                elif not self.model_microbatch_after_dp:
                    best = new_best
            return best, final[0], final[1], final[2], vtp, flags, None

        costs, plans, remains, mems, flags = solve(list(range(S)), strategy_set)
        best, vtp = pick_vtp(costs, plans, np.inf)
        if vtp != -1:
            return best, [p[vtp] for p in plans], [r[vtp] for r in remains], [m[vtp] for m in mems], vtp, flags, None
        return best, None, [-1] * len(remains), [-1] * len(mems), vtp, flags, None

    # ------------------------------------------------------------------ all pipeline degrees
    def fit(self, bsz, min_tp, max_tp, vsp, embed_sdp, sp_search, print_=True, mbsz_dict=None):
        best = dict(cost=np.inf, plan=None, pp=-1, remain=-1, mem=-1, vtp=-1)
        if mbsz_dict is None:
            mbsz_dict = {pp: 8 for pp in self.ppdeg_set}

        def say(msg):
            if not print_:
                return
            if self.logger is not None:
                self.logger.info(msg)
            else:
                print(msg, flush=True)

        for pp_deg in self.ppdeg_set:
            if pp_deg * min_tp > self.gpu_num:
                continue
            say(f"bsz={bsz}, pp_deg={pp_deg}, min_tp={min_tp}, max_tp={max_tp}, vsp={vsp}, embed_sdp={embed_sdp}, sp_search={sp_search}:")
            if bsz % (self.gpu_num // (pp_deg * min_tp)):
                if best["plan"] is None:
                    best["plan"] = "[current bsz is not divisible by bsz_scale]"
                say("Best strategy: False \nFrom history: False")
                say(f"time cost: {np.inf}, memory remaining: -1, memory cost: {np.inf}")
                continue
            assert self.multi_layer_type
            cost, plan, remain, mem, vtp, flags, hist = self._build_dp_and_run_multi_layer_type(
                pp_deg, bsz, mbsz_dict[pp_deg], min_tp, max_tp, vsp, embed_sdp, sp_search)
            mem = [m + self.mem_cache for m in mem] if isinstance(mem, list) else mem + self.mem_cache
            say(f"Best strategy: {flags} \nFrom history: {hist}")
            say(f"time cost: {cost}, memory remaining: {remain}, memory cost: {mem}")
            if best["cost"] > cost:
                best = dict(cost=cost, plan=plan, pp=pp_deg, remain=remain, mem=mem, vtp=vtp)
        return best["cost"], best["plan"], best["pp"], best["remain"], best["mem"], best["vtp"]
