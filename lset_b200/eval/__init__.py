from .chunked_encoder import encode_chunked
from .mteb_evaluator import LSETMTEBModel

__all__ = ["LSETMTEBModel", "encode_chunked"]
