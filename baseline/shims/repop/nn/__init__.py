"""`repop.nn`: modules and functional ops of the model forward and backward."""
