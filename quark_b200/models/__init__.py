from .waypoint_15 import GenerateFrame, QuantConfig, TransformerBlock, Waypoint15, Waypoint15Config, make_params  # noqa: F401
