from .distributions import Uniform, Bernoulli, Binomial, Categorical, Normal  # noqa: F401
from .kl_losses import (  # noqa: F401
    kl_normal_normal, kl_normal_standard, kl_bernoulli_bernoulli, kl_categorical_categorical,
    kl_uniform_uniform, kl_div_loss, js_divergence,
)
from .kl_losses import (  # noqa: F401,E402
    kl_normal_normal_scalar, kl_normal_normal_diag, kl_bernoulli_scalar, kl_bernoulli_vector, kl_categorical,
    kl_divergence, kl_divergence_any, kl_normal_normal_diag_sum, kl_normal_normal_diag_batched,
    kl_bernoulli_sum, kl_bernoulli_batched, kl_categorical_sum, kl_categorical_batched,
)
