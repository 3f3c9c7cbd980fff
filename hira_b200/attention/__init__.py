from .hira_attention import hira_attention, hira_decode_attention

__all__ = ["hira_attention", "hira_decode_attention"]
