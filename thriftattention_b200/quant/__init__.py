from .formats import Mxfp4QuantFormat, Nvfp4QuantFormat, QuantFormat, get_quant_format

__all__ = ["Mxfp4QuantFormat", "Nvfp4QuantFormat", "QuantFormat", "get_quant_format"]
