"""Batch optimizers for ``--search iterative``.

An optimizer proposes a batch of samples (``suggest``), is told the score of
each (``observe``; the score is the fraction of peak, higher is better) and is
closed with ``finished``.  The interface and the preset names are the
reference's (``itf/search/optimizer.py``, ``search/optimizers.py:20-236``):

``random``                     draws from the strategy's sampler;
``random-forest-default``      a random-forest surrogate over the sample vector,
``random-forest-explore``      ranked by an upper confidence bound
``random-forest-aggressive``   ``(mean - best) + beta * std`` over the trees, with
                               ``beta`` decaying as ``beta0 / n_observed ** alpha``
                               down to a floor of 0.05.

Presets differ in ``beta0``, ``alpha`` and the forest's size and depth; a YAML
file given as ``config_file`` overrides single keys.  The forest is refitted
each time ``update_period`` more observations have arrived, never before
``update_first`` of them.  The kernels' spaces are small (at most a few hundred
legal samples), so candidates a strategy hands out twice are proposed once and
samples already observed are not proposed again while unseen ones remain.
"""

from __future__ import annotations

import logging
import random
from typing import Any, Callable, Sequence

import numpy as np

logger = logging.getLogger(__name__)

VecSample = list[int]
SampleFn = Callable[[int, int], Sequence[VecSample]]


class Optimizer:
    """``suggest`` / ``observe`` / ``finished``."""

    def __init__(self, sample_fn: SampleFn, batch: int, seed: int) -> None:
        self.sample_fn = sample_fn
        self.batch = max(int(batch), 1)
        self.rng = random.Random(seed)
        self.X: list[VecSample] = []
        self.y: list[float] = []
        self.best_x: VecSample = []
        self.best_y = 0.0

    def draw(self, num: int) -> list[VecSample]:
        """``num`` samples from the strategy with a fresh seed, duplicates removed."""
        out: list[VecSample] = []
        seen: set[tuple[int, ...]] = set()
        for s in self.sample_fn(num, self.rng.randint(0, 2**32 - 1)):
            key = tuple(int(v) for v in s)
            if key not in seen:
                seen.add(key)
                out.append(list(key))
        return out

    def unseen_first(self, candidates: list[VecSample]) -> list[VecSample]:
        done = {tuple(x) for x in self.X}
        fresh = [c for c in candidates if tuple(c) not in done]
        return fresh if fresh else candidates

    def suggest(self) -> list[VecSample]:
        raise NotImplementedError

    def observe(self, x: Sequence[VecSample], y: Sequence[float]) -> None:
        assert len(x) == len(y), "one score per sample"
        for xi, yi in zip(x, y):
            self.X.append([int(v) for v in xi])
            self.y.append(float(yi))
            if yi > self.best_y:
                self.best_x, self.best_y = list(xi), float(yi)

    def finished(self) -> None:
        logger.info("optimizer: %d observations, best %.4f at %s", len(self.y), self.best_y, self.best_x)


class RandomOptimizer(Optimizer):
    def __init__(self, sample_fn: SampleFn, batch: int, seed: int, **_unused: Any) -> None:
        super().__init__(sample_fn, batch, seed)

    def suggest(self) -> list[VecSample]:
        return self.unseen_first(self.draw(self.batch))[: self.batch]


class RandomForestOptimizer(Optimizer):
    BETA_FLOOR = 0.05

    def __init__(self, sample_fn: SampleFn, batch: int, seed: int, *, batch_candidates: int = 1000,
                 beta: float = 2.5, alpha: float = 0.7, update_first: int | None = None,
                 update_period: int | None = None, n_estimators: int = 300, max_depth: int = 12,
                 min_samples_leaf: int = 5, max_features: float = 0.8) -> None:
        super().__init__(sample_fn, batch, seed)
        from sklearn.ensemble import RandomForestRegressor

        self.batch_candidates = int(batch_candidates)
        self.beta0 = float(beta)
        self.alpha = float(alpha)
        self.update_first = int(update_first) if update_first else self.batch
        self.update_period = int(update_period) if update_period else self.batch
        self.fitted_on = 0
        self.last_beta: float | None = None
        self.forest = RandomForestRegressor(
            n_estimators=n_estimators, n_jobs=1, max_depth=max_depth,
            min_samples_leaf=min_samples_leaf, min_samples_split=2 * min_samples_leaf,
            max_features=max_features, random_state=seed)

    def beta(self) -> float:
        return max(self.BETA_FLOOR, self.beta0 / max(len(self.y), 1) ** self.alpha)

    def scores(self, candidates: list[VecSample]) -> np.ndarray:
        per_tree = np.stack([t.predict(np.asarray(candidates, dtype=float))
                             for t in self.forest.estimators_])
        self.last_beta = self.beta()
        return (per_tree.mean(axis=0) - self.best_y) + self.last_beta * per_tree.std(axis=0)

    def suggest(self) -> list[VecSample]:
        candidates = self.unseen_first(self.draw(self.batch_candidates))
        if not self.fitted_on:
            self.rng.shuffle(candidates)
            return candidates[: self.batch]
        order = np.argsort(-self.scores(candidates), kind="stable")
        return [candidates[i] for i in order[: self.batch]]

    def observe(self, x: Sequence[VecSample], y: Sequence[float]) -> None:
        super().observe(x, y)
        n = len(self.X)
        if n < self.update_first:
            return
        due = self.update_first + (n - self.update_first) // self.update_period * self.update_period
        if due > self.fitted_on:
            self.forest.fit(np.asarray(self.X[:due], dtype=float), np.asarray(self.y[:due]))
            self.fitted_on = due


PRESETS: dict[str, tuple[type[Optimizer], dict[str, Any]]] = {
    "random": (RandomOptimizer, {}),
    "random-forest-default": (RandomForestOptimizer, dict(
        batch_candidates=1000, beta=2.5, alpha=0.7, n_estimators=300, max_depth=12,
        min_samples_leaf=5, max_features=0.8)),
    "random-forest-explore": (RandomForestOptimizer, dict(
        batch_candidates=1000, beta=5.0, alpha=0.6, n_estimators=300, max_depth=10,
        min_samples_leaf=3, max_features=0.9)),
    "random-forest-aggressive": (RandomForestOptimizer, dict(
        batch_candidates=1000, beta=2.0, alpha=0.8, n_estimators=200, max_depth=8,
        min_samples_leaf=5, max_features=0.7)),
}


class Optimizers:
    """Name -> optimizer registry."""

    @classmethod
    def names(cls) -> list[str]:
        return list(PRESETS)

    @classmethod
    def create(cls, name: str, sample_fn: SampleFn, batch: int, seed: int,
               config_file: str | None = None) -> Optimizer:
        if name not in PRESETS:
            raise ValueError(f"unknown optimizer name: {name}")
        kind, preset = PRESETS[name]
        options = dict(preset)
        if config_file:
            import yaml

            with open(config_file) as f:
                options.update(yaml.safe_load(f) or {})
        return kind(sample_fn, batch, seed, **options)
