/*
 * Source compatibility with code written against the reference library's C API: include this header instead of
 * smem.h / smem_bm.h / smem_shm.h / smem_trans.h / hybm*.h and the reference's names resolve to this library's functions,
 * types and enumerators (reference headers: src/smem/include/host/*.h, src/hybm/include/*.h). Only names are mapped;
 * semantics are those documented in the mf_*.h headers.
 */
#ifndef MF_PUBLIC_SMEM_COMPAT_H
#define MF_PUBLIC_SMEM_COMPAT_H

#include "mf.h"
#include "mf_bm.h"
#include "mf_hybm.h"
#include "mf_shm.h"
#include "mf_trans.h"

/* ---- common ---- */
#define ASYNC_COPY_FLAG MF_ASYNC_COPY_FLAG
#define COPY_EXTEND_FLAG MF_COPY_KERNEL_FLAG
#define SMEM_WORLD_SIZE_MAX MF_WORLD_SIZE_MAX
#define SMEM_INVALID_DEV_ID MF_INVALID_DEV_ID
#define SM_OK MF_OK
#define SM_ERROR MF_ERROR
#define SM_INVALID_PARAM MF_INVALID_PARAM
#define SM_MALLOC_FAILED MF_MALLOC_FAILED
#define SM_NEW_OBJECT_FAILED MF_NEW_OBJECT_FAILED
#define SM_NOT_STARTED MF_NOT_STARTED
#define SM_TIMEOUT MF_TIMEOUT
#define SM_REPEAT_CALL MF_REPEAT_CALL
#define SM_DUPLICATED_OBJECT MF_DUPLICATED_OBJECT
#define SM_OBJECT_NOT_EXISTS MF_OBJECT_NOT_EXISTS
#define SM_NOT_INITIALIZED MF_NOT_INITIALIZED
#define SM_RESOURCE_IN_USE MF_RESOURCE_IN_USE
#define SM_RECONNECT MF_RECONNECT
#define SM_GET_OBJIECT MF_GET_OBJECT
#define smem_tls_config mf_tls_config
#define smem_decrypt_handler mf_decrypt_handler

/* ---- common functions ---- */
#define smem_create_config_store mf_create_config_store
#define smem_get_and_clear_last_err_msg mf_get_and_clear_last_err_msg
#define smem_get_last_err_msg mf_get_last_err_msg
#define smem_init mf_init
#define smem_set_conf_store_tls mf_set_conf_store_tls
#define smem_set_config_store_tls_key mf_set_config_store_tls_key
#define smem_set_extern_logger mf_set_extern_logger
#define smem_set_log_level mf_set_log_level
#define smem_uninit mf_uninit

/* ---- BM ---- */
#define smem_bm_config_init mf_bm_config_init
#define smem_bm_copy mf_bm_copy
#define smem_bm_copy_batch mf_bm_copy_batch
#define smem_bm_copy_batch_on_stream mf_bm_copy_batch_on_stream
#define smem_bm_copy_on_stream mf_bm_copy_on_stream
#define smem_bm_create mf_bm_create
#define smem_bm_create2 mf_bm_create2
#define smem_bm_destroy mf_bm_destroy
#define smem_bm_get_joined_size mf_bm_get_joined_size
#define smem_bm_get_local_mem_size_by_mem_type mf_bm_get_local_mem_size_by_mem_type
#define smem_bm_get_rank_id mf_bm_get_rank_id
#define smem_bm_get_rank_id_by_gva mf_bm_get_rank_id_by_gva
#define smem_bm_init mf_bm_init
#define smem_bm_join mf_bm_join
#define smem_bm_leave mf_bm_leave
#define smem_bm_ptr_by_mem_type mf_bm_ptr_by_mem_type
#define smem_bm_register_user_mem mf_bm_register_user_mem
#define smem_bm_uninit mf_bm_uninit
#define smem_bm_unregister_user_mem mf_bm_unregister_user_mem
#define smem_bm_wait mf_bm_wait

/* ---- SHM ---- */
#define smem_shm_atomic_alloc_value mf_shm_atomic_alloc_value
#define smem_shm_atomic_release_value mf_shm_atomic_release_value
#define smem_shm_config_init mf_shm_config_init
#define smem_shm_control_allgather mf_shm_control_allgather
#define smem_shm_control_barrier mf_shm_control_barrier
#define smem_shm_create mf_shm_create
#define smem_shm_destroy mf_shm_destroy
#define smem_shm_get_device_meta mf_shm_get_device_meta
#define smem_shm_get_global_rank mf_shm_get_global_rank
#define smem_shm_get_global_rank_size mf_shm_get_global_rank_size
#define smem_shm_get_multicast_ptr mf_shm_get_multicast_ptr
#define smem_shm_get_signal_base mf_shm_get_signal_base
#define smem_shm_global_exit mf_shm_global_exit
#define smem_shm_init mf_shm_init
#define smem_shm_next_epoch mf_shm_next_epoch
#define smem_shm_query_support_data_operation mf_shm_query_support_data_operation
#define smem_shm_register_exit mf_shm_register_exit
#define smem_shm_set_extra_context mf_shm_set_extra_context
#define smem_shm_subgroup_allgather mf_shm_subgroup_allgather
#define smem_shm_subgroup_barrier mf_shm_subgroup_barrier
#define smem_shm_topology_can_reach mf_shm_topology_can_reach
#define smem_shm_uninit mf_shm_uninit

/* ---- TRANS ---- */
#define smem_trans_batch_read mf_trans_batch_read
#define smem_trans_batch_read_submit mf_trans_batch_read_submit
#define smem_trans_batch_register_mem mf_trans_batch_register_mem
#define smem_trans_batch_write mf_trans_batch_write
#define smem_trans_batch_write_submit mf_trans_batch_write_submit
#define smem_trans_config_init mf_trans_config_init
#define smem_trans_create mf_trans_create
#define smem_trans_deregister_mem mf_trans_deregister_mem
#define smem_trans_destroy mf_trans_destroy
#define smem_trans_free mf_trans_free
#define smem_trans_get_rank mf_trans_get_rank
#define smem_trans_init mf_trans_init
#define smem_trans_malloc mf_trans_malloc
#define smem_trans_read mf_trans_read
#define smem_trans_read_submit mf_trans_read_submit
#define smem_trans_register_mem mf_trans_register_mem
#define smem_trans_uninit mf_trans_uninit
#define smem_trans_write mf_trans_write
#define smem_trans_write_submit mf_trans_write_submit

/* ---- hybm core ---- */
#define hybm_alloc_local_memory mf_hybm_alloc_local_memory
#define hybm_create_entity mf_hybm_create_entity
#define hybm_data_batch_copy mf_hybm_data_batch_copy
#define hybm_data_copy mf_hybm_data_copy
#define hybm_destroy_entity mf_hybm_destroy_entity
#define hybm_entity_reach_types mf_hybm_entity_reach_types
#define hybm_export mf_hybm_export
#define hybm_export_slice_size mf_hybm_export_slice_size
#define hybm_free_local_memory mf_hybm_free_local_memory
#define hybm_get_device_meta mf_hybm_get_device_meta
#define hybm_get_error_string mf_hybm_get_error_string
#define hybm_get_memory_ptr mf_hybm_get_memory_ptr
#define hybm_get_slice_va mf_hybm_get_slice_va
#define hybm_import mf_hybm_import
#define hybm_init mf_hybm_init
#define hybm_mmap mf_hybm_mmap
#define hybm_register_local_memory mf_hybm_register_local_memory
#define hybm_remove_imported mf_hybm_remove_imported
#define hybm_reserve_mem_space mf_hybm_reserve_mem_space
#define hybm_reserve_mem_space_at mf_hybm_reserve_mem_space_at
#define hybm_set_extern_logger mf_hybm_set_extern_logger
#define hybm_set_extra_context mf_hybm_set_extra_context
#define hybm_set_log_level mf_hybm_set_log_level
#define hybm_uninit mf_hybm_uninit
#define hybm_unmap mf_hybm_unmap
#define hybm_unreserve_mem_space mf_hybm_unreserve_mem_space
#define hybm_wait mf_hybm_wait

/* ---- types and enumerators ---- */
#define smem_bm_t mf_bm_t
#define smem_bm_config_t mf_bm_config_t
#define smem_bm_create_option_t mf_bm_create_option_t
#define smem_copy_params mf_copy_params
#define smem_batch_copy_params mf_batch_copy_params
#define smem_bm_mem_type mf_bm_mem_type
#define smem_bm_data_op_type mf_bm_data_op_type
#define smem_bm_copy_type mf_bm_copy_type
#define SMEM_MEM_TYPE_LOCAL_DEVICE MF_MEM_TYPE_LOCAL_DEVICE
#define SMEM_MEM_TYPE_LOCAL_HOST MF_MEM_TYPE_LOCAL_HOST
#define SMEM_MEM_TYPE_DEVICE MF_MEM_TYPE_DEVICE
#define SMEM_MEM_TYPE_HOST MF_MEM_TYPE_HOST
#define SMEMB_DATA_OP_SDMA MF_BM_DATA_OP_SDMA
#define SMEMB_DATA_OP_HOST_RDMA MF_BM_DATA_OP_HOST_RDMA
#define SMEMB_DATA_OP_HOST_TCP MF_BM_DATA_OP_HOST_TCP
#define SMEMB_DATA_OP_DEVICE_RDMA MF_BM_DATA_OP_DEVICE_RDMA
#define SMEMB_DATA_OP_HOST_URMA MF_BM_DATA_OP_HOST_URMA
#define SMEMB_COPY_L2G MF_BM_COPY_L2G
#define SMEMB_COPY_G2L MF_BM_COPY_G2L
#define SMEMB_COPY_G2H MF_BM_COPY_G2H
#define SMEMB_COPY_H2G MF_BM_COPY_H2G
#define SMEMB_COPY_L2GH MF_BM_COPY_L2GH
#define SMEMB_COPY_GH2L MF_BM_COPY_GH2L
#define SMEMB_COPY_GH2H MF_BM_COPY_GH2H
#define SMEMB_COPY_H2GH MF_BM_COPY_H2GH
#define SMEMB_COPY_G2G MF_BM_COPY_G2G
#define SMEMB_COPY_AUTO MF_BM_COPY_AUTO
#define SMEM_BM_FLAG_CREATE_WITH_SHM MF_BM_FLAG_CREATE_WITH_SHM
#define smem_shm_t mf_shm_t
#define smem_shm_config_t mf_shm_config_t
#define smem_shm_data_op_type mf_shm_data_op_type
#define SMEMS_DATA_OP_MTE MF_SHM_DATA_OP_MTE
#define SMEMS_DATA_OP_SDMA MF_SHM_DATA_OP_SDMA
#define SMEMS_DATA_OP_RDMA MF_SHM_DATA_OP_RDMA
#define smem_trans_t mf_trans_t
#define smem_trans_config_t mf_trans_config_t
#define smem_trans_role_t mf_trans_role_t
#define SMEM_TRANS_NONE MF_TRANS_NONE
#define SMEM_TRANS_SENDER MF_TRANS_SENDER
#define SMEM_TRANS_RECEIVER MF_TRANS_RECEIVER
#define SMEM_TRANS_BOTH MF_TRANS_BOTH
#define hybm_entity_t mf_hybm_entity_t
#define hybm_mem_slice_t mf_hybm_mem_slice_t
#define hybm_options mf_hybm_options
#define hybm_exchange_info mf_hybm_exchange_info
#define hybm_copy_params mf_hybm_copy_params
#define hybm_batch_copy_params mf_hybm_batch_copy_params

#endif
