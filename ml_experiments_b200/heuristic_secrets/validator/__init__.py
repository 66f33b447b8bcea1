from .features import (FeatureSet, FrequencyTable, char_frequency_difference, char_type_mix, extract_features,  # noqa: F401
                       kolmogorov_complexity, shannon_entropy)
from .model import ValidatorConfig, ValidatorModel  # noqa: F401
