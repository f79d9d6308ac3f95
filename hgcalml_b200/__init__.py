"""hgcalml_b200: sm_100a CUDA kernels behind the HGCalML GravNet / object-condensation ops.

The modules mirror the reference's Python wrappers by name (``bin_by_coordinates_op``,
``binned_select_knn_op``, ``accknn_op``, ``index_replacer_op``, ``assign_condensate_op``, ``local_distance_op``, ``push_knn_op``,
``GravNetLayersRagged``); they take
torch CUDA tensors and call the C ABI of ``libhgcalml_b200.so``.  Importing an op module without
the built library raises ImportError: there is no CPU or eager fallback.
"""
__version__ = "0.1.0"
