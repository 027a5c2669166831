from .engine import Engine, ServeConfig, Scheduler, paged_decode_attention, greedy_sample
