"""Test infrastructure: CPU restatement of the reference's token loop and the
recipe that rebuilds the reference itself.  Never imported by the product."""
