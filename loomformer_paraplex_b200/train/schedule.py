"""Learning-rate schedule: linear warm-up then cosine decay to ``min_lr_frac`` of the peak
(reference ``loomformer.py:4136-4142``)."""
import math


def lr_at(cfg, step_zero_based: int) -> float:
    if step_zero_based < cfg.warmup_steps:
        return cfg.lr * (step_zero_based + 1) / max(1, cfg.warmup_steps)
    prog = (step_zero_based - cfg.warmup_steps) / max(1, cfg.steps - cfg.warmup_steps)
    prog = min(1.0, max(0.0, prog))
    return cfg.lr * (cfg.min_lr_frac + (1.0 - cfg.min_lr_frac) * 0.5 * (1.0 + math.cos(math.pi * prog)))
