// Native helper of OutputDiscardCheckpoint: make a tensor whose storage was emptied see the bytes of a freshly
// recomputed tensor WITHOUT copying them and WITHOUT replacing the tensor's StorageImpl.
//
// Autograd-saved references to the discarded tensor (and every view of it) hold the same StorageImpl, so the only
// way they can all see the recomputed data for free is to swap the allocation underneath that StorageImpl. The
// recomputed tensor's StorageImpl keeps owning the allocation; the emptied one borrows the pointer through a
// DataPtr whose context holds a strong reference to the owner, which is dropped when the borrower lets go.
// Same contract as src/olmo_core/nn/_csrc/share_storage.cpp:12-30 of the reference; registered as a dispatcher op
// (torch.ops.ocb_native.rebind_storage) and compiled ahead of time instead of at first use.

#include <ATen/ATen.h>
#include <torch/library.h>

namespace {

struct OwnerRef {
    c10::intrusive_ptr<c10::StorageImpl> owner;
};

void drop_owner(void* ctx) { delete static_cast<OwnerRef*>(ctx); }

void rebind_storage(const at::Tensor& dst, const at::Tensor& src) {
    TORCH_CHECK(dst.defined() && src.defined(), "rebind_storage: undefined tensor");
    TORCH_CHECK(dst.device() == src.device(), "rebind_storage: tensors live on different devices");
    c10::StorageImpl* borrower = dst.storage().unsafeGetStorageImpl();
    c10::StorageImpl* lender = src.storage().unsafeGetStorageImpl();
    if (borrower == lender) return;
    TORCH_CHECK(static_cast<size_t>(dst.storage_offset() + dst.numel()) * dst.element_size() <= lender->nbytes(),
                "rebind_storage: the recomputed storage is smaller than the discarded tensor");
    auto keep = c10::intrusive_ptr<c10::StorageImpl>::reclaim_copy(lender);
    void* bytes = keep->mutable_data();
    const size_t nbytes = keep->nbytes();
    const c10::Device device = keep->device();
    borrower->set_data_ptr_noswap(c10::DataPtr(bytes, new OwnerRef{std::move(keep)}, &drop_owner, device));
    borrower->set_nbytes(nbytes);
}

}  // namespace

TORCH_LIBRARY(ocb_native, m) {
    m.def("rebind_storage(Tensor dst, Tensor src) -> ()", &rebind_storage);
}
