from .distributions import Uniform, Bernoulli, Binomial, Categorical, Normal  # noqa: F401
from .kl_losses import (  # noqa: F401
    kl_normal_normal, kl_normal_standard, kl_bernoulli_bernoulli, kl_categorical_categorical,
    kl_uniform_uniform, kl_div_loss, js_divergence,
)
