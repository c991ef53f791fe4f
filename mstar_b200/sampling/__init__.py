from .params import SamplingParams, seed_from_request_id

__all__ = ["SamplingParams", "seed_from_request_id"]
