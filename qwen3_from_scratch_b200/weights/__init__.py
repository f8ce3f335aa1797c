from .loader import WeightsError, load_weights  # noqa: F401
from .random_init import random_weights_on_device, write_random_model  # noqa: F401
from .specs import model_weight_specs  # noqa: F401
