"""CPU oracle - TEST INFRASTRUCTURE, not part of the product.  See nabla_oracle.c."""
