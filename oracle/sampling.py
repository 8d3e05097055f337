"""TEST INFRASTRUCTURE — pure-Python oracle of the reference's host-side sampler and
DFlash accept-prefix decision.  Never imported by the product.

Restates, operation by operation in f64:
  * crates/qwen-llm/src/sampling.rs — `SamplingConfig::validate` (:133-144),
    `Sampler::{new, at_draw, sample, diagnose, couple_deterministic_proposal,
    couple_sparse_proposal}` (:340-367, :377-399, :530-603 via the
    candidate-vector formulation `reference_sample` :605-688, :692-790),
    `candidate_order` (:1110-1115), `greedy_token` (:1159-1181),
    `probability_weights` (:1515-1539), `diagnose_candidates` (:1541-1614),
    `Xoshiro256PlusPlus` / `SplitMix64` (:1619-1670);
  * crates/qwen-llm/src/metal_dflash/accept.rs — `decide_dflash_accept_prefix`
    (:76-183).
Pinned by the reference's golden vectors (sampling.rs:1817-1878) and its eight
accept-prefix tests (accept.rs:236-616); see tests/test_oracle_sampling.py.
"""
from __future__ import annotations

import copy
import math
import struct
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

MASK64 = (1 << 64) - 1


class SamplingError(Exception):
    def __init__(self, kind: str, detail=None):
        super().__init__(f"{kind}: {detail}")
        self.kind = kind
        self.detail = detail


def _f32(x: float) -> float:
    """Round a Python float to the nearest binary32 (as the reference's f32 fields do)."""
    return struct.unpack("<f", struct.pack("<f", x))[0]


def _f32_bits(x: float) -> int:
    return struct.unpack("<I", struct.pack("<f", x))[0]


class SplitMix64:
    def __init__(self, seed: int):
        self.s = seed & MASK64

    def next(self) -> int:
        self.s = (self.s + 0x9E3779B97F4A7C15) & MASK64
        v = self.s
        v = ((v ^ (v >> 30)) * 0xBF58476D1CE4E5B9) & MASK64
        v = ((v ^ (v >> 27)) * 0x94D049BB133111EB) & MASK64
        return v ^ (v >> 31)


def _rotl(x: int, k: int) -> int:
    return ((x << k) | (x >> (64 - k))) & MASK64


class Xoshiro256PlusPlus:
    def __init__(self, seed: int):
        sm = SplitMix64(seed)
        self.state = [sm.next(), sm.next(), sm.next(), sm.next()]

    def next_u64(self) -> int:
        s = self.state
        result = (_rotl((s[0] + s[3]) & MASK64, 23) + s[0]) & MASK64
        t = (s[1] << 17) & MASK64
        s[2] ^= s[0]
        s[3] ^= s[1]
        s[1] ^= s[2]
        s[0] ^= s[3]
        s[2] ^= t
        s[3] = _rotl(s[3], 45)
        return result

    def next_unit_f64(self) -> float:
        return float(self.next_u64() >> 11) / float(1 << 53)


@dataclass
class SamplingConfig:
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    min_p: float = 0.0
    seed: int = 0

    def validate(self) -> "SamplingConfig":
        t, p, m = self.temperature, self.top_p, self.min_p
        if not math.isfinite(t) or t < 0.0:
            raise SamplingError("InvalidTemperature", t)
        if not math.isfinite(p) or not (0.0 < p <= 1.0):
            raise SamplingError("InvalidTopP", p)
        if not math.isfinite(m) or not (0.0 <= m <= 1.0):
            raise SamplingError("InvalidMinP", m)
        return SamplingConfig(_f32(t), int(self.top_k), _f32(p), _f32(m), self.seed & MASK64)


def _order_key(token: int, logit: float) -> Tuple[int, int]:
    """Ascending sort key equal to `candidate_order`: logit descending in f32 total
    order (so +0.0 before -0.0), then token ascending."""
    bits = _f32_bits(logit)
    ascending = (~bits & 0xFFFFFFFF) if bits & 0x80000000 else (bits | 0x80000000)
    return ((~ascending) & 0xFFFFFFFF, token)


def greedy_token(logits: Sequence[float]) -> int:
    n = len(logits)
    if n == 0:
        raise SamplingError("EmptyLogits")
    best, best_logit = 0, float(logits[0])
    if math.isnan(best_logit):
        raise SamplingError("NanLogit", 0)
    best_key = _order_key(0, best_logit)[0]
    for token in range(1, n):
        l = float(logits[token])
        if math.isnan(l):
            raise SamplingError("NanLogit", token)
        k = _order_key(token, l)[0]
        if k < best_key:  # strictly greater in total order
            best, best_key = token, k
    return best


def _sorted_candidates(logits: Sequence[float], top_k: int) -> List[List]:
    n = len(logits)
    if n == 0:
        raise SamplingError("EmptyLogits")
    cands = []
    for token in range(n):
        l = float(logits[token])
        if math.isnan(l):
            raise SamplingError("NanLogit", token)
        cands.append((_order_key(token, l), token, l))
    cands.sort(key=lambda c: c[0])
    if 0 < top_k < n:
        cands = cands[:top_k]
    return [[c[1], c[2]] for c in cands]  # [token, f64 logit]


def _probability_weights(cands: List[List]) -> List[float]:
    if any(c[1] == math.inf for c in cands):
        return [1.0 if c[1] == math.inf else 0.0 for c in cands]
    max_logit = cands[0][1]
    if max_logit == -math.inf:
        raise SamplingError("NoCandidates")
    weights = []
    for c in cands:
        try:
            w = math.exp(c[1] - max_logit)
        except OverflowError:
            w = math.inf
        weights.append(w)
    if any(not math.isfinite(w) for w in weights):
        raise SamplingError("NoCandidates")
    return weights


@dataclass
class Distribution:
    candidates: List[Tuple[int, float]]  # (token, weight) in categorical order
    total_weight: float
    token: int
    candidate_index: int


def _diagnose_candidates(cfg: SamplingConfig, cands: List[List], uniform: float) -> Distribution:
    if cfg.min_p > 0.0:
        max_logit = cands[0][1]
        if math.isfinite(max_logit):
            threshold = max_logit + math.log(cfg.min_p)
            cands = [c for c in cands if c[1] >= threshold]
    if not cands:
        raise SamplingError("NoCandidates")
    if cands[0][1] == math.inf:
        cands = [c for c in cands if c[1] == math.inf]
    t = cfg.temperature
    cands = [[c[0], c[1] / t] for c in cands]
    weights = _probability_weights(cands)
    if cfg.top_p < 1.0:
        total = 0.0
        for w in weights:
            total += w
        target = total * cfg.top_p
        cum, keep = 0.0, 0
        for w in weights:
            cum += w
            keep += 1
            if cum >= target:
                break
        keep = max(keep, 1)
        cands, weights = cands[:keep], weights[:keep]
    total_weight = 0.0
    for w in weights:
        total_weight += w
    if not (math.isfinite(total_weight) and total_weight > 0.0):
        raise SamplingError("NoCandidates")
    target = uniform * total_weight
    cum, idx = 0.0, len(cands) - 1
    for i, w in enumerate(weights):
        cum += w
        if target < cum:
            idx = i
            break
    return Distribution([(c[0], w) for c, w in zip(cands, weights)], total_weight, cands[idx][0], idx)


@dataclass
class SparseProposal:
    token: int
    candidates: List[Tuple[int, float]] = field(default_factory=list)  # (token, weight)


class Sampler:
    def __init__(self, config: SamplingConfig):
        self.config = config.validate()
        self.rng = Xoshiro256PlusPlus(self.config.seed)
        self.draws = 0

    @classmethod
    def at_draw(cls, config: SamplingConfig, draws: int) -> "Sampler":
        s = cls(config)
        for _ in range(draws):
            s.rng.next_u64()
        s.draws = draws
        return s

    def clone(self) -> "Sampler":
        return copy.deepcopy(self)

    def diagnose(self, logits, uniform: float) -> Distribution:
        if self.config.temperature == 0.0:
            tok = greedy_token(logits)
            return Distribution([(tok, 1.0)], 1.0, tok, 0)
        return _diagnose_candidates(self.config, _sorted_candidates(logits, self.config.top_k), uniform)

    def sample(self, logits) -> Tuple[int, int]:
        """Returns (token, candidate_index); one RNG draw per successful positive-temperature call."""
        if self.config.temperature == 0.0:
            return greedy_token(logits), 0
        cands = _sorted_candidates(logits, self.config.top_k)
        # Build the distribution with a placeholder draw first so that an error consumes no RNG state.
        probe = _diagnose_candidates(self.config, cands, 0.0)
        self.draws += 1
        target = self.rng.next_unit_f64() * probe.total_weight
        cum, idx = 0.0, len(probe.candidates) - 1
        for i, (_, w) in enumerate(probe.candidates):
            cum += w
            if target < cum:
                idx = i
                break
        return probe.candidates[idx][0], idx

    def sample_with_distribution(self, logits) -> Distribution:
        """sampling.rs:437-452: the draw together with the filtered categorical distribution it was made from;
        an error leaves the generator untouched."""
        if self.config.temperature == 0.0:
            return self.diagnose(logits, 0.0)
        probe = copy.deepcopy(self.rng)
        dist = self.diagnose(logits, probe.next_unit_f64())
        self.rng = probe
        self.draws += 1
        return dist

    def couple_deterministic_proposal(self, logits, proposal: int):
        target, _ = self.sample(logits)
        return ("accepted", None) if target == proposal else ("rejected", target)

    def couple_sparse_proposal(self, logits, proposal: SparseProposal):
        n = len(logits)
        if proposal.token < 0 or proposal.token >= n:
            raise SamplingError("ProposalTokenOutOfRange", proposal.token)
        if not proposal.candidates:
            raise SamplingError("NoCandidates")
        proposal_total = 0.0
        proposal_token_weight = 0.0
        for tok, w in proposal.candidates:
            if tok < 0 or tok >= n:
                raise SamplingError("ProposalTokenOutOfRange", tok)
            if not math.isfinite(w) or w < 0.0:
                raise SamplingError("InvalidProposalWeight", (tok, w))
            proposal_total += w
            if tok == proposal.token:
                proposal_token_weight += w
        if not (math.isfinite(proposal_total) and proposal_total > 0.0):
            raise SamplingError("NoCandidates")
        if not (math.isfinite(proposal_token_weight) and proposal_token_weight > 0.0):
            raise SamplingError("MissingProposalToken", proposal.token)
        target = self.diagnose(logits, 0.0)
        s = 0.0
        for tok, w in target.candidates:
            if tok == proposal.token:
                s += w
        target_probability = s / target.total_weight
        proposal_probability = proposal_token_weight / proposal_total
        acceptance = min(target_probability / proposal_probability, 1.0)
        self.draws += 1
        if self.rng.next_unit_f64() < acceptance:
            return ("accepted", None)
        residual = []
        residual_total = 0.0
        for tok, w in target.candidates:
            tp = w / target.total_weight
            ps = 0.0
            for ptok, pw in proposal.candidates:
                if ptok == tok:
                    ps += pw
            pp = ps / proposal_total
            rw = max(tp - pp, 0.0)
            residual_total += rw
            residual.append((tok, rw))
        if not (math.isfinite(residual_total) and residual_total > 0.0):
            raise SamplingError("NoCandidates")
        self.draws += 1
        threshold = self.rng.next_unit_f64() * residual_total
        cum = 0.0
        for tok, rw in residual:
            cum += rw
            if threshold < cum:
                return ("rejected", tok)
        return ("rejected", residual[-1][0])


# ---------------------------------------------------------------------------
# accept.rs:76-183
# ---------------------------------------------------------------------------
class AcceptError(Exception):
    def __init__(self, kind: str, detail=None, row: Optional[int] = None):
        super().__init__(f"{kind}: {detail} (row {row})")
        self.kind = kind
        self.detail = detail
        self.row = row


@dataclass
class AcceptDecision:
    accepted_drafts: List[int]
    next_carry: Optional[Tuple[str, int]]  # ("correction"|"bonus", token)
    stop_reason: Optional[str]             # "eos" | "token_limit"
    retain_input_count: int


def decide_dflash_accept_prefix(verified_tokens: Sequence[int], target_logits: Sequence[float], vocab: int,
                                proposals: Optional[Sequence[SparseProposal]], sampler: Sampler,
                                remaining_output_budget: int, stop_ids: Sequence[int]) -> AcceptDecision:
    if len(verified_tokens) == 0:
        raise AcceptError("InvalidInput", "missing carry token")
    if vocab == 0 or vocab > 0x7FFFFFFF:
        raise AcceptError("InvalidInput", "invalid vocabulary size")
    if len(verified_tokens) * vocab != len(target_logits):
        raise AcceptError("InvalidInput", "target logits extent mismatch")
    for index, token in enumerate(verified_tokens):
        if token < 0 or token >= vocab:
            raise AcceptError("InvalidToken", (index, token, vocab))
    n_drafts = len(verified_tokens) - 1
    if proposals is not None:
        if len(proposals) != n_drafts:
            raise AcceptError("InvalidInput", "proposal row count mismatch")
        for row, proposal in enumerate(proposals):
            draft = verified_tokens[row + 1]
            if proposal.token != draft:
                raise AcceptError("ProposalMismatch", (row, proposal.token, draft))
            for tok, _ in proposal.candidates:
                if tok < 0 or tok >= vocab:
                    raise AcceptError("Sampling", "ProposalTokenOutOfRange", row)
    if verified_tokens[0] in stop_ids:
        return AcceptDecision([], None, "eos", 0)
    if remaining_output_budget == 0:
        return AcceptDecision([], None, "token_limit", 0)

    nxt = sampler.clone()
    accepted: List[int] = []
    next_carry, stop_reason = None, None
    while True:
        row = len(accepted)
        logits = target_logits[row * vocab:(row + 1) * vocab]
        try:
            if row == n_drafts:
                bonus, _ = nxt.sample(logits)
                next_carry = ("bonus", bonus)
                break
            draft = verified_tokens[row + 1]
            if proposals is not None:
                decision = nxt.couple_sparse_proposal(logits, proposals[row])
            else:
                decision = nxt.couple_deterministic_proposal(logits, draft)
        except SamplingError as e:
            raise AcceptError("Sampling", e.kind, row)
        if decision[0] == "rejected":
            next_carry = ("correction", decision[1])
            break
        accepted.append(draft)
        if draft in stop_ids:
            stop_reason = "eos"
            break
        if len(accepted) == remaining_output_budget:
            stop_reason = "token_limit"
            break
    retain = 1 + len(accepted) - (1 if stop_reason is not None else 0)
    sampler.rng = nxt.rng
    sampler.draws = nxt.draws
    return AcceptDecision(accepted, next_carry, stop_reason, retain)
