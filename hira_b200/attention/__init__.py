from .hira_attention import (HiraDecodeStep, hira_attention, hira_decode_attention, make_hira_attention,
                             register_hira_attention)

__all__ = ["HiraDecodeStep", "hira_attention", "hira_decode_attention", "make_hira_attention", "register_hira_attention"]
