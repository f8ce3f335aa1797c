from .loader import WeightsError, load_weights  # noqa: F401
from .random_init import write_random_model  # noqa: F401
from .specs import model_weight_specs  # noqa: F401
